// FlashDeformAttn backward: grad_value (scatter), grad of the sampling locations and of the
// attention logits (softmax Jacobian applied in-kernel).
//
// Replaces backward_kernel_warp_primitive / backward_kernel + launchers
// (DCNv4_op/src/cuda/flash_deform_col2im_cuda.cuh:20-580) and the zero-fills / fp16 casts
// of DCNv4_op/src/cuda/flash_deform_attn_cuda.cu:125-131,157-162.
//
// Same structure as the DCNv4 backward (a lane owns 4 channels): vector reductions into an
// fp32 grad_value buffer, shuffle reduction of the per-point partials over a pair's lanes,
// gradient rows assembled in shared memory and written out whole; persistent CTAs with a
// double-buffered bulk-copy stage.  The logit gradient uses
//   grad_logit_i = p_i * (g_i - sum_j g_j p_j),
// which equals the reference's explicit Jacobian loop; a point that fails the range test
// contributes g = 0 (the reference reads a never-written shared-memory slot there).
#include "common.cuh"

namespace dcnb200 {

size_t fda_bwd_smem(const FdaParams& p, int elem) {
  const size_t n = (size_t)p.tile * p.G * 3 * p.LK;
  const size_t span = (n * elem + 15) & ~(size_t)15;
  const size_t gsz = (n * sizeof(float) + 15) & ~(size_t)15;
  return 16 + 2 * span + gsz + (size_t)p.tile * p.G * sizeof(float2);
}

// DETR: 4 levels x 4 points and one chunk per lane as compile-time constants (see fda_fwd.cu).
template <typename T, int V, bool DETR>
__global__ void __launch_bounds__(kThreads, DCNB200_BWD_MINB)
fda_bwd_kernel(const T* __restrict__ value, const int64_t* __restrict__ shapes,
               const int64_t* __restrict__ starts, const T* __restrict__ sla,
               const T* __restrict__ gout, float* __restrict__ gvalue, T* __restrict__ gsla,
               const FdaParams p, int* status) {
  constexpr int VS = 16 / (int)sizeof(T);  // elements per 16-byte store of the write-out
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int s_lvl[kMaxLevels * 3];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw);
  const int rowlen = p.G * 3 * p.LK;
  const size_t sbytes = ((size_t)p.tile * rowlen * sizeof(T) + 15) & ~(size_t)15;
  const size_t gbytes = ((size_t)p.tile * rowlen * sizeof(float) + 15) & ~(size_t)15;
  T* s_buf[2] = {reinterpret_cast<T*>(smem_raw + 16), reinterpret_cast<T*>(smem_raw + 16 + sbytes)};
  float* s_g = reinterpret_cast<float*>(smem_raw + 16 + 2 * sbytes);
  float2* s_stat = reinterpret_cast<float2*>(smem_raw + 16 + 2 * sbytes + gbytes);
  const int n_tiles = (p.nq + p.tile - 1) / p.tile;

  auto issue = [&](int tile, int buf) {
    const int q0 = tile * p.tile;
    const int nq_tile = min(p.tile, p.nq - q0);
    issue_stage(s_buf[buf], sla + (size_t)q0 * rowlen, (uint32_t)(nq_tile * rowlen * sizeof(T)), 1, 0, 0, &bar[buf]);
  };

  if (threadIdx.x < p.L) load_level(&s_lvl[threadIdx.x * 3], shapes, starts, (int)threadIdx.x, p.Len_in, status);
  if (threadIdx.x == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
  }
  __syncthreads();
  // Tiles are dealt round-robin: at any moment the CTAs work on neighbouring tiles, i.e. on the
  // same image, so that image's value tensor (and in the backward its fp32 gradient accumulator,
  // the target of the reductions) is what occupies L2 -- with contiguous shares every CTA would
  // be in a different image and the working set (all images) would not fit.  Sampling locations
  // are arbitrary, so unlike DCNv4 there is no L1 locality between neighbouring tiles to keep.
  const int tile_begin = (int)blockIdx.x, tile_step = (int)gridDim.x, tile_end = n_tiles;
  if (threadIdx.x == 0 && tile_begin < tile_end) issue(tile_begin, 0);

  const int LK = p.LK;
  const int tpg = p.tpg_b;
  const int tpg_shift = 31 - __clz(tpg);

  int it = 0;
  for (int tile = tile_begin; tile < tile_end; tile += tile_step, ++it) {
    const int cur = it & 1;
    const int next = tile + tile_step;
    if (threadIdx.x == 0 && next < tile_end) issue(next, cur ^ 1);
    const int q0 = tile * p.tile;
    const int nq_tile = min(p.tile, p.nq - q0);
    T* s_row = s_buf[cur];
    copy_tail(s_row, sla + (size_t)q0 * rowlen, (uint32_t)(nq_tile * rowlen * sizeof(T)));
    wait_stage(&bar[cur], (uint32_t)((it >> 1) & 1), status);
    __syncthreads();

    for (int pr = threadIdx.x; pr < nq_tile * p.G; pr += kThreads) {
      const T* lg = s_row + pr * 3 * LK + 2 * LK;
      float mx = -INFINITY;
      for (int t = 0; t < LK; ++t) mx = fmaxf(mx, to_f32(lg[t]));
      float sum = 0.f;
      for (int t = 0; t < LK; ++t) sum += __expf(to_f32(lg[t]) - mx);
      s_stat[pr] = make_float2(mx, 1.f / sum);
    }
    __syncthreads();

    const int n_items = nq_tile * p.G * tpg;
    for (int base = 0; base < n_items; base += kThreads) {
      const bool active = base + threadIdx.x < n_items;
      const int item = active ? base + threadIdx.x : 0;
      const int c = item & (tpg - 1);
      const int pr = item >> tpg_shift;
      const int ql = fast_div(pr, p.div_g);
      const int g = pr - ql * p.G;
      const int q = q0 + ql;
      const int b = q / p.Len_q;
      const T* row = s_row + pr * 3 * LK;
      float* grow = s_g + pr * 3 * LK;
      const float2 stat = s_stat[pr];
      const T* go_ptr = gout + (size_t)q * p.C + g * p.D + c * V;
      float gy0[V];
      gather_corner<T, V>(go_ptr, active, gy0);

      float dot = 0.f;  // sum_t g_t p_t, kept by lane 0 of the pair
      const int n_lvl = DETR ? 4 : p.L, n_pts = DETR ? 4 : p.K, n_chunks = DETR ? 1 : p.chunks_b;
#pragma unroll(DETR ? 4 : 1)
      for (int l = 0; l < n_lvl; ++l) {
        const int Hl = s_lvl[l * 3], Wl = s_lvl[l * 3 + 1];
        const float Hf = (float)Hl, Wf = (float)Wl;
        const size_t img_off = ((size_t)b * p.Len_in + s_lvl[l * 3 + 2]) * p.C + g * p.D + c * V;
#pragma unroll(DETR ? 4 : 2)
        for (int k = 0; k < n_pts; ++k) {
          const int t = l * n_pts + k;
          const float w_im = fda_coord(to_f32(row[2 * t]), Wf);
          const float h_im = fda_coord(to_f32(row[2 * t + 1]), Hf);
          const float m = __expf(to_f32(row[2 * LK + t]) - stat.x) * stat.y;
          float gx = 0.f, gyv = 0.f, gm = 0.f;
          bool ok = bwd_point<T, V>(value + img_off, gvalue + img_off, Hl, Wl, p.C, Hf, Wf, h_im, w_im, m, active,
                                    gy0, gx, gyv, gm);
          for (int ci = 1; ci < n_chunks; ++ci) {
            const int off = ci * tpg * V;
            float gy[V];
            gather_corner<T, V>(go_ptr + off, active, gy);
            ok = bwd_point<T, V>(value + img_off + off, gvalue + img_off + off, Hl, Wl, p.C, Hf, Wf, h_im, w_im, m,
                                 active, gy, gx, gyv, gm);
          }
          for (int o = tpg >> 1; o > 0; o >>= 1) {
            gx += __shfl_xor_sync(0xffffffffu, gx, o);
            gyv += __shfl_xor_sync(0xffffffffu, gyv, o);
            gm += __shfl_xor_sync(0xffffffffu, gm, o);
          }
          if (active && c == 0) {
            grow[2 * t] = ok ? Wf * m * gx : 0.f;
            grow[2 * t + 1] = ok ? Hf * m * gyv : 0.f;
            const float gt = ok ? gm : 0.f;
            grow[2 * LK + t] = gt;
            dot = fmaf(gt, m, dot);
          }
        }
      }
      if (active && c == 0) {
        for (int t = 0; t < LK; ++t) {
          const float m = __expf(to_f32(row[2 * LK + t]) - stat.x) * stat.y;
          grow[2 * LK + t] = m * (grow[2 * LK + t] - dot);
        }
      }
    }

    __syncthreads();
    // write the tile's gradient rows: 16-byte vectors, then a ragged tail element by element
    const int n_elem = nq_tile * rowlen;
    const int n_vec = n_elem / VS;
    T* dst = gsla + (size_t)q0 * rowlen;
    for (int i = threadIdx.x; i < n_vec; i += kThreads) {
      float v[VS];
#pragma unroll
      for (int e = 0; e < VS; e += 4) {
        const float4 f4 = *reinterpret_cast<const float4*>(s_g + (size_t)i * VS + e);
        v[e] = f4.x; v[e + 1] = f4.y; v[e + 2] = f4.z; v[e + 3] = f4.w;
      }
      uint32_t packed[4];
      narrow(v, packed, (const T*)nullptr);
      stg_raw(dst + (size_t)i * VS, packed);
    }
    for (int i = n_vec * VS + threadIdx.x; i < n_elem; i += kThreads) dst[i] = from_f32<T>(s_g[i]);
    __syncthreads();  // s_g, statistics and this staging buffer are free for the next tile
  }
}

template <typename T, int V>
static cudaError_t launch_v(const T* value, const int64_t* shapes, const int64_t* starts, const T* sla,
                            const T* gout, float* gvalue, T* gsla, const FdaParams& p, int* status,
                            cudaStream_t s) {
  const size_t smem = fda_bwd_smem(p, sizeof(T));
  const bool detr = p.L == 4 && p.K == 4 && p.chunks_b == 1;
  auto kern = detr ? fda_bwd_kernel<T, V, true> : fda_bwd_kernel<T, V, false>;
  int per_sm = 1;
  cudaError_t e = detr ? persistent_ctas_per_sm<fda_bwd_kernel<T, V, true>>(smem, &per_sm)
                       : persistent_ctas_per_sm<fda_bwd_kernel<T, V, false>>(smem, &per_sm);
  if (e != cudaSuccess) return e;
  const long long n_tiles = ((long long)p.nq + p.tile - 1) / p.tile;
  const long long want = (long long)p.sm_count * per_sm;
  kern<<<(int)(n_tiles < want ? n_tiles : want), kThreads, smem, s>>>(value, shapes, starts, sla, gout, gvalue,
                                                                     gsla, p, status);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_t(const T* value, const int64_t* shapes, const int64_t* starts, const T* sla,
                            const T* gout, float* gvalue, T* gsla, const FdaParams& p, int* status,
                            cudaStream_t s) {
  return p.lane_ch_b == 8 ? launch_v<T, 8>(value, shapes, starts, sla, gout, gvalue, gsla, p, status, s)
                          : launch_v<T, 4>(value, shapes, starts, sla, gout, gvalue, gsla, p, status, s);
}

cudaError_t launch_fda_bwd(int dtype, const void* value, const int64_t* shapes, const int64_t* starts,
                           const void* sla, const void* gout, float* gvalue_f32, void* gsla,
                           const FdaParams& p, int* status, cudaStream_t s) {
  switch (dtype) {
    case 0: return launch_t((const float*)value, shapes, starts, (const float*)sla, (const float*)gout, gvalue_f32, (float*)gsla, p, status, s);
    case 1: return launch_t((const __half*)value, shapes, starts, (const __half*)sla, (const __half*)gout, gvalue_f32, (__half*)gsla, p, status, s);
    default: return launch_t((const __nv_bfloat16*)value, shapes, starts, (const __nv_bfloat16*)sla, (const __nv_bfloat16*)gout, gvalue_f32, (__nv_bfloat16*)gsla, p, status, s);
  }
}

}  // namespace dcnb200
