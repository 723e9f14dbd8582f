// FlashDeformAttn forward: softmax over the L*K logits of a (query, head), then the
// probability-weighted sum of bilinear samples taken from L feature levels.
//
// Replaces forward_kernel_reg + launchers
// (DCNv4_op/src/cuda/flash_deform_im2col_cuda.cuh:129-451) and the zero-filled output of
// DCNv4_op/src/cuda/flash_deform_attn_cuda.cu:60.
//
// The softmax statistics (max, 1/sum) are computed once per (query, head) while the tile is
// in shared memory -- not once per channel lane -- and the level table (H_l, W_l, start_l)
// is read from device memory once per CTA instead of once per thread and level.
#include "common.cuh"

namespace dcnb200 {

size_t fda_fwd_smem(const FdaParams& p, int elem) {
  const size_t row = ((size_t)p.tile * p.G * 3 * p.LK * elem + 15) & ~(size_t)15;
  return 16 + row + (size_t)p.tile * p.G * sizeof(float2);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
fda_fwd_kernel(const T* __restrict__ value, const int64_t* __restrict__ shapes,
               const int64_t* __restrict__ starts, const T* __restrict__ sla, T* __restrict__ out,
               const FdaParams p, int* status) {
  constexpr int V = Vec<T>::N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int s_lvl[kMaxLevels * 3];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw);
  T* s_row = reinterpret_cast<T*>(smem_raw + 16);
  const int rowlen = p.G * 3 * p.LK;  // elements per query
  const size_t row_bytes = ((size_t)p.tile * rowlen * sizeof(T) + 15) & ~(size_t)15;
  float2* s_stat = reinterpret_cast<float2*>(smem_raw + 16 + row_bytes);

  const int q0 = blockIdx.x * p.tile;
  const int nq_tile = min(p.tile, p.nq - q0);
  if (threadIdx.x < p.L) {
    s_lvl[threadIdx.x * 3] = (int)shapes[threadIdx.x * 2];
    s_lvl[threadIdx.x * 3 + 1] = (int)shapes[threadIdx.x * 2 + 1];
    s_lvl[threadIdx.x * 3 + 2] = (int)starts[threadIdx.x];
  }
  if (!stage_span(s_row, sla + (size_t)q0 * rowlen, (uint32_t)(nq_tile * rowlen * sizeof(T)), bar, status)) return;

  const int LK = p.LK;
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
    const int c = item % p.tpg;
    const int pr = item / p.tpg;
    const int g = pr % p.G;
    const int ql = pr / p.G;
    const int q = q0 + ql;
    const int b = q / p.Len_q;
    const T* row = s_row + pr * 3 * LK;
    const float2 stat = s_stat[pr];

    for (int ci = 0; ci < p.chunks; ++ci) {
      const int ch0 = (c + ci * p.tpg) * V;
      float acc[V];
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] = 0.f;
      for (int l = 0; l < p.L; ++l) {
        const int Hl = s_lvl[l * 3], Wl = s_lvl[l * 3 + 1];
        const T* img = value + ((size_t)b * p.Len_in + s_lvl[l * 3 + 2]) * p.C + g * p.D + ch0;
#pragma unroll 4
        for (int k = 0; k < p.K; ++k) {
          const int t = l * p.K + k;
          const float w_im = fda_coord(to_f32(row[2 * t]), Wl);
          const float h_im = fda_coord(to_f32(row[2 * t + 1]), Hl);
          const float m = __expf(to_f32(row[2 * LK + t]) - stat.x) * stat.y;
          const bool ok = in_range(h_im, w_im, Hl, Wl);
          const Footprint f = footprint(h_im, w_im, Hl, Wl);
          const T* p1 = img + ((ptrdiff_t)f.h0 * Wl + f.w0) * p.C;
          const uint4 r1 = ldg_vec(p1, ok && f.top && f.left);
          const uint4 r2 = ldg_vec(p1 + p.C, ok && f.top && f.right);
          const uint4 r3 = ldg_vec(p1 + (size_t)Wl * p.C, ok && f.bot && f.left);
          const uint4 r4 = ldg_vec(p1 + (size_t)Wl * p.C + p.C, ok && f.bot && f.right);
          const float w1 = m * f.hh * f.hw, w2 = m * f.hh * f.lw, w3 = m * f.lh * f.hw, w4 = m * f.lh * f.lw;
          float v1[V], v2[V], v3[V], v4[V];
          unpack(r1, v1, (const T*)nullptr);
          unpack(r2, v2, (const T*)nullptr);
          unpack(r3, v3, (const T*)nullptr);
          unpack(r4, v4, (const T*)nullptr);
#pragma unroll
          for (int e = 0; e < V; ++e)
            acc[e] = fmaf(w1, v1[e], fmaf(w2, v2[e], fmaf(w3, v3[e], fmaf(w4, v4[e], acc[e]))));
        }
      }
      *reinterpret_cast<uint4*>(out + (size_t)q * p.C + g * p.D + ch0) = pack(acc, (const T*)nullptr);
    }
  }
}

template <typename T>
static cudaError_t launch_t(const T* value, const int64_t* shapes, const int64_t* starts, const T* sla,
                            T* out, const FdaParams& p, int* status, cudaStream_t s) {
  const int grid = (p.nq + p.tile - 1) / p.tile;
  fda_fwd_kernel<T><<<grid, kThreads, fda_fwd_smem(p, sizeof(T)), s>>>(value, shapes, starts, sla, out, p, status);
  return cudaGetLastError();
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
