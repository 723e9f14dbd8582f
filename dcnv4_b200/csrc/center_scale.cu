// Centre-feature-scale blend of the DCNv4 module in one pass:
//     s[r, g]   = sigmoid( sum_c x[r, c] * weight[g, c] + bias[g] )           one scale per row and group
//     out[r, c] = x[r, c] * (1 - s[r, c / D]) + x_proj[r, c] * s[r, c / D]
// where x is the operator's output and x_proj its input (the value projection).  The reference
// runs this as a Linear, a sigmoid, a repeat, two multiplies and an add
// (DCNv4_op/DCNv4/modules/dcnv4.py:18-26,142-147); none of its CUDA sources covers it.
//
// A warp owns a row: every lane keeps its 16-byte vectors of the row in registers (fp32), the G dot
// products are accumulated against weight rows read through L1 (lanes read consecutive vectors, so the
// weight loads are coalesced and shared by all warps of the SM), each is folded with five shuffles,
// lane 0 applies bias and sigmoid and leaves the scale in a per-warp shared-memory slot, and the blend is
// written with the same 16-byte vectors.  Arithmetic is fp32, one rounding on store.
#include "common.cuh"

namespace dcnb200 {

constexpr int kCsMaxVec = 8;     // 16-byte vectors a lane may hold
constexpr int kCsMaxGroups = 128;
constexpr int kCsWarps = 8;

template <typename T, typename P, int NV>
__global__ void __launch_bounds__(kCsWarps * 32)
center_scale_blend_kernel(const T* __restrict__ x, const T* __restrict__ xp, const P* __restrict__ weight,
                          const P* __restrict__ bias, T* __restrict__ out, long long rows, int C, int G, int D) {
  constexpr int E = 16 / (int)sizeof(T);
  __shared__ float s_scale[kCsWarps][kCsMaxGroups];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long gwarp = (long long)blockIdx.x * kCsWarps + warp;
  const long long n_warps = (long long)gridDim.x * kCsWarps;
  pdl_trigger();
  pdl_wait();  // x and x_proj are previous kernels' outputs
  for (long long row = gwarp; row < rows; row += n_warps) {
    float xv[NV][E];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c0 = (lane + v * 32) * E;
      const RawVec<16> raw = ldg_raw<16>(x + row * C + c0, c0 < C);
      widen(raw.r, xv[v], (const T*)nullptr);
    }
    for (int g = 0; g < G; ++g) {
      const P* wrow = weight + (size_t)g * C;
      float acc = 0.f;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c0 = (lane + v * 32) * E;
        if (c0 < C) {
#pragma unroll
          for (int e = 0; e < E; ++e) acc = fmaf(xv[v][e], to_f32(wrow[c0 + e]), acc);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) s_scale[warp][g] = 1.f / (1.f + __expf(-(acc + to_f32(bias[g]))));
    }
    __syncwarp();
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c0 = (lane + v * 32) * E;
      if (c0 < C) {
        const float s = s_scale[warp][c0 / D];   // D is a multiple of E: a vector lies inside one group
        const RawVec<16> raw = ldg_raw<16>(xp + row * C + c0, true);
        float pv[E], o[E];
        widen(raw.r, pv, (const T*)nullptr);
#pragma unroll
        for (int e = 0; e < E; ++e) o[e] = fmaf(pv[e], s, xv[v][e] * (1.f - s));
        uint32_t packed[4];
        narrow(o, packed, (const T*)nullptr);
        stg_raw(out + row * C + c0, packed);
      }
    }
    __syncwarp();  // the scale slots are rewritten for the next row
  }
}

template <typename T, typename P>
static cudaError_t launch_tp(const T* x, const T* xp, const P* w, const P* b, T* out, long long rows, int G, int D,
                             int sm_count, cudaStream_t s) {
  constexpr int E = 16 / (int)sizeof(T);
  const int C = G * D;
  const int nv = (C / E + 31) / 32;
  long long blocks = (rows + kCsWarps - 1) / kCsWarps;
  const long long cap = (long long)(sm_count > 0 ? sm_count : 1) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
#define CS_CASE(NVV) \
  case NVV: return launch_overlapped(center_scale_blend_kernel<T, P, NVV>, dim3((unsigned)blocks), dim3(kCsWarps * 32), 0, s, x, xp, w, b, out, rows, C, G, D);
  switch (nv) {
    CS_CASE(1) CS_CASE(2) CS_CASE(3) CS_CASE(4) CS_CASE(5) CS_CASE(6) CS_CASE(7) CS_CASE(8)
    default: return cudaErrorInvalidValue;
  }
#undef CS_CASE
}

int center_scale_max_channels(int dtype) { return 32 * kCsMaxVec * (dtype == 0 ? 4 : 8); }
int center_scale_max_groups() { return kCsMaxGroups; }

// dtype / param_dtype: 0 fp32, 1 fp16, 2 bf16; parameters are either fp32 or the tensor's own type.
cudaError_t launch_center_scale_blend(int dtype, int param_dtype, const void* x, const void* xp, const void* w,
                                      const void* b, void* out, long long rows, int G, int D, int sm_count,
                                      cudaStream_t s) {
  const bool pf32 = param_dtype == 0;
  switch (dtype) {
    case 0:
      return launch_tp((const float*)x, (const float*)xp, (const float*)w, (const float*)b, (float*)out, rows, G, D, sm_count, s);
    case 1:
      return pf32 ? launch_tp((const __half*)x, (const __half*)xp, (const float*)w, (const float*)b, (__half*)out, rows, G, D, sm_count, s)
                  : launch_tp((const __half*)x, (const __half*)xp, (const __half*)w, (const __half*)b, (__half*)out, rows, G, D, sm_count, s);
    default:
      return pf32 ? launch_tp((const __nv_bfloat16*)x, (const __nv_bfloat16*)xp, (const float*)w, (const float*)b, (__nv_bfloat16*)out, rows, G, D, sm_count, s)
                  : launch_tp((const __nv_bfloat16*)x, (const __nv_bfloat16*)xp, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, rows, G, D, sm_count, s);
  }
}

}  // namespace dcnb200
