// FlashDeformAttn forward: softmax over the L*K logits of a (query, head), then the
// probability-weighted sum of bilinear samples taken from L feature levels.
//
// Replaces forward_kernel_reg + launchers
// (DCNv4_op/src/cuda/flash_deform_im2col_cuda.cuh:129-451) and the zero-filled output of
// DCNv4_op/src/cuda/flash_deform_attn_cuda.cu:60.
//
// A lane owns 32 bytes of channels (one 256-bit load per corner).  The softmax statistics (max, 1/sum) are computed once per (query, head) while the tile is
// in shared memory -- not once per channel lane -- and the level table (H_l, W_l, start_l)
// is read from device memory once per CTA instead of once per thread and level.
#include "common.cuh"

namespace dcnb200 {

size_t fda_fwd_smem(const FdaParams& p, int elem) {
  const size_t row = ((size_t)p.tile * p.G * 3 * p.LK * elem + 15) & ~(size_t)15;
  return 16 + row + (size_t)p.tile * p.G * sizeof(float2);
}

template <typename T, int VB>
__global__ void __launch_bounds__(kThreads, 2)
fda_fwd_kernel(const T* __restrict__ value, const int64_t* __restrict__ shapes,
               const int64_t* __restrict__ starts, const T* __restrict__ sla, T* __restrict__ out,
               const FdaParams p, int* status) {
  constexpr int V = VB / (int)sizeof(T);
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
  if (!stage_rows(s_row, sla + (size_t)q0 * rowlen, (uint32_t)(nq_tile * rowlen * sizeof(T)), 1, 0, 0, bar, status))
    return;

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
        const float Hf = (float)Hl, Wf = (float)Wl;
        const T* img = value + ((size_t)b * p.Len_in + s_lvl[l * 3 + 2]) * p.C + g * p.D + ch0;
#pragma unroll 4
        for (int k = 0; k < p.K; ++k) {
          const int t = l * p.K + k;
          const float w_im = fda_coord(to_f32(row[2 * t]), Wf);
          const float h_im = fda_coord(to_f32(row[2 * t + 1]), Hf);
          const float m = __expf(to_f32(row[2 * LK + t]) - stat.x) * stat.y;
          fwd_point<T, VB>(img, Hl, Wl, p.C, h_im, w_im, m, acc);
        }
      }
      uint32_t packed[VB / 4];
      narrow(acc, packed, (const T*)nullptr);
      stg_raw(out + (size_t)q * p.C + g * p.D + ch0, packed);
    }
  }
}

template <typename T>
static cudaError_t launch_t(const T* value, const int64_t* shapes, const int64_t* starts, const T* sla,
                            T* out, const FdaParams& p, int* status, cudaStream_t s) {
  const int grid = (p.nq + p.tile - 1) / p.tile;
  const size_t smem = fda_fwd_smem(p, sizeof(T));
  if (p.vb == 32)
    fda_fwd_kernel<T, 32><<<grid, kThreads, smem, s>>>(value, shapes, starts, sla, out, p, status);
  else
    fda_fwd_kernel<T, 16><<<grid, kThreads, smem, s>>>(value, shapes, starts, sla, out, p, status);
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
