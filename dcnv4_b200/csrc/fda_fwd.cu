// FlashDeformAttn forward: softmax over the L*K logits of a (query, head), then the
// probability-weighted sum of bilinear samples taken from L feature levels.
//
// Replaces forward_kernel_reg + launchers
// (DCNv4_op/src/cuda/flash_deform_im2col_cuda.cuh:129-451) and the zero-filled output of
// DCNv4_op/src/cuda/flash_deform_attn_cuda.cu:60.
//
// Persistent CTAs loop over tiles of consecutive queries; a tile's packed location/logit rows
// are one contiguous span staged with a bulk copy into a double-buffered shared-memory
// stage.  A lane owns 32 bytes of a head's channels.  The softmax statistics (max, 1/sum) are
// computed once per (query, head) while the tile is in shared memory -- not once per channel
// lane -- and the level table (H_l, W_l, start_l) is read from device memory once per CTA
// instead of once per thread and level.
#include "common.cuh"

namespace dcnb200 {

static size_t span_bytes(const FdaParams& p, int elem) {
  return ((size_t)p.tile * p.G * 3 * p.LK * elem + 15) & ~(size_t)15;
}

size_t fda_fwd_smem(const FdaParams& p, int elem) {
  return 16 + 2 * span_bytes(p, elem) + (size_t)p.tile * p.G * sizeof(float2);
}

// DETR: the Deformable-DETR configuration (4 levels x 4 points, all channels of a lane in one
// chunk) as compile-time constants -- the level and point loops unroll fully and the row offsets
// become immediates; every other configuration takes the generic path of the same kernel.
template <typename T, int V, bool DETR>
__global__ void __launch_bounds__(kThreads, DCNB200_FWD_MINB)
fda_fwd_kernel(const T* __restrict__ value, const int64_t* __restrict__ shapes,
               const int64_t* __restrict__ starts, const T* __restrict__ sla, T* __restrict__ out,
               const FdaParams p, int* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int s_lvl[kMaxLevels * 3];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw);
  const int rowlen = p.G * 3 * p.LK;  // elements per query
  const size_t sbytes = ((size_t)p.tile * rowlen * sizeof(T) + 15) & ~(size_t)15;
  T* s_buf[2] = {reinterpret_cast<T*>(smem_raw + 16), reinterpret_cast<T*>(smem_raw + 16 + sbytes)};
  float2* s_stat = reinterpret_cast<float2*>(smem_raw + 16 + 2 * sbytes);
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
  const int tpg_shift = 31 - __clz(p.tpg);

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
    __syncthreads();  // the tail (if any) is visible to every thread

    for (int pr = threadIdx.x; pr < nq_tile * p.G; pr += kThreads) {
      const T* lg = s_row + pr * 3 * LK + 2 * LK;
      float mx = -INFINITY;
      for (int t = 0; t < LK; ++t) mx = fmaxf(mx, to_f32(lg[t]));
      float sum = 0.f;
      for (int t = 0; t < LK; ++t) sum += __expf(to_f32(lg[t]) - mx);
      s_stat[pr] = make_float2(mx, 1.f / sum);
    }
    __syncthreads();

    const int n_items = nq_tile * p.G * p.tpg;
    for (int item = threadIdx.x; item < n_items; item += kThreads) {
      const int c = item & (p.tpg - 1);
      const int pr = item >> tpg_shift;
      const int ql = fast_div(pr, p.div_g);
      const int g = pr - ql * p.G;
      const int q = q0 + ql;
      const int b = q / p.Len_q;
      const T* row = s_row + pr * 3 * LK;
      const float2 stat = s_stat[pr];

      const int n_chunks = DETR ? 1 : p.chunks, n_lvl = DETR ? 4 : p.L, n_pts = DETR ? 4 : p.K;
      for (int ci = 0; ci < n_chunks; ++ci) {
        const int ch0 = (c + ci * p.tpg) * V;
        float acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = 0.f;
#pragma unroll(DETR ? 4 : 1)
        for (int l = 0; l < n_lvl; ++l) {
          const int Hl = s_lvl[l * 3], Wl = s_lvl[l * 3 + 1];
          const float Hf = (float)Hl, Wf = (float)Wl;
          const T* img = value + ((size_t)b * p.Len_in + s_lvl[l * 3 + 2]) * p.C + g * p.D + ch0;
#pragma unroll 4
          for (int k = 0; k < n_pts; ++k) {
            const int t = l * n_pts + k;
            const float w_im = fda_coord(to_f32(row[2 * t]), Wf);
            const float h_im = fda_coord(to_f32(row[2 * t + 1]), Hf);
            const float m = __expf(to_f32(row[2 * LK + t]) - stat.x) * stat.y;
            fwd_point<T, V>(img, Hl, Wl, p.C, Hf, Wf, h_im, w_im, m, acc);
          }
        }
        constexpr int WORDS = V * (int)sizeof(T) / 4;
        uint32_t packed[WORDS];
        narrow(acc, packed, (const T*)nullptr);
        T* dst = out + (size_t)q * p.C + g * p.D + ch0;
        if constexpr (WORDS == 16) {
          uint32_t lo[8], hi[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) { lo[e] = packed[e]; hi[e] = packed[8 + e]; }
          stg_raw(dst, lo);
          stg_raw(dst + V / 2, hi);
        } else {
          stg_raw(dst, packed);
        }
      }
    }
    __syncthreads();  // buffer and statistics are free for the tile after next
  }
}

template <typename T, int V>
static cudaError_t launch_v(const T* value, const int64_t* shapes, const int64_t* starts, const T* sla,
                            T* out, const FdaParams& p, int* status, cudaStream_t s) {
  const size_t smem = fda_fwd_smem(p, sizeof(T));
  const bool detr = p.L == 4 && p.K == 4 && p.chunks == 1;
  auto kern = detr ? fda_fwd_kernel<T, V, true> : fda_fwd_kernel<T, V, false>;
  int per_sm = 1;
  cudaError_t e = detr ? persistent_ctas_per_sm<fda_fwd_kernel<T, V, true>>(smem, &per_sm)
                       : persistent_ctas_per_sm<fda_fwd_kernel<T, V, false>>(smem, &per_sm);
  if (e != cudaSuccess) return e;
  const long long n_tiles = ((long long)p.nq + p.tile - 1) / p.tile;
  const long long want = (long long)p.sm_count * per_sm;
  kern<<<(int)(n_tiles < want ? n_tiles : want), kThreads, smem, s>>>(value, shapes, starts, sla, out, p, status);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_t(const T* value, const int64_t* shapes, const int64_t* starts, const T* sla,
                            T* out, const FdaParams& p, int* status, cudaStream_t s) {
  const int bytes = p.lane_ch * (int)sizeof(T);
  if constexpr (sizeof(T) == 4) {
    if (bytes == 64) return launch_v<T, 16>(value, shapes, starts, sla, out, p, status, s);
  }
  if (bytes == 32) return launch_v<T, 32 / (int)sizeof(T)>(value, shapes, starts, sla, out, p, status, s);
  return launch_v<T, 16 / (int)sizeof(T)>(value, shapes, starts, sla, out, p, status, s);
}

cudaError_t launch_fda_fwd(int dtype, const void* value, const int64_t* shapes, const int64_t* starts,
                           const void* sla, void* out, const FdaParams& p, int* status, cudaStream_t s) {
  switch (dtype) {
    case 0: return launch_t((const float*)value, shapes, starts, (const float*)sla, (float*)out, p, status, s);
    case 1: return launch_t((const __half*)value, shapes, starts, (const __half*)sla, (__half*)out, p, status, s);
    default: return launch_t((const __nv_bfloat16*)value, shapes, starts, (const __nv_bfloat16*)sla, (__nv_bfloat16*)out, p, status, s);
  }
}

}  // namespace dcnb200
