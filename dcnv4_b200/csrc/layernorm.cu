// Channels-last LayerNorm forward for the FlashInternImage blocks around the DCNv4 operator.
//
// The model normalises rows of C = 64..1280 contiguous channels (N*H*W rows).  A framework kernel that
// gives a whole thread block to such a short row spends its time on launch geometry, not on memory:
// in FlashInternImage-T fp16 inference the stock LayerNorm was more than half of the GPU time.  Here a
// row is owned by LPR = 2..32 adjacent lanes (16 bytes per lane and step), a warp handles 32/LPR rows
// at once, statistics are two shuffle reductions in fp32 over register-resident data, and each element
// is read and written exactly once: the kernel runs at HBM speed.
//
// The reference builds these norms from torch.nn.LayerNorm (classification/models/flash_intern_image.py:34-56);
// this kernel has no counterpart among its CUDA sources.
#include "common.cuh"

namespace dcnb200 {

constexpr int kLnMaxVec = 8;  // 16-byte vectors a lane may hold (C <= 32 lanes * 8 vectors * elements per vector)

// GELU in the erf form of torch.nn.GELU(), evaluated in fp32.
__device__ __forceinline__ float gelu_erf(float v) { return 0.5f * v * (1.f + erff(v * 0.70710678118654752f)); }

// GELU: apply the activation to the normalised value after it has been rounded to the storage type
// (what a separate LayerNorm and GELU pair computes), then round again.
template <typename T, typename P, int NV, bool GELU>
__global__ void __launch_bounds__(256)
layernorm_fwd_kernel(const T* __restrict__ x, const P* __restrict__ gamma, const P* __restrict__ beta,
                     T* __restrict__ y, long long rows, int C, int lpr, float eps) {
  constexpr int E = 16 / (int)sizeof(T);  // elements per 16-byte vector
  const int lane = threadIdx.x & 31;
  const int sub = lane % lpr;             // lane within the row
  const int rows_per_warp = 32 / lpr;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const float inv_c = 1.f / (float)C;

  pdl_trigger();
  pdl_wait();  // x -- and the parameters, e.g. after a fold or an optimiser step -- may be a previous kernel's output

  // this lane's slice of gamma / beta: vectors sub, sub + lpr, ...
  float g[NV][E], b[NV][E];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c0 = (sub + v * lpr) * E;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const bool ok = c0 + e < C;
      g[v][e] = ok ? to_f32(gamma[c0 + e]) : 0.f;
      b[v][e] = ok ? to_f32(beta[c0 + e]) : 0.f;
    }
  }
  for (long long r0 = warp * rows_per_warp; r0 < rows; r0 += n_warps * rows_per_warp) {
    const long long row = r0 + lane / lpr;
    const bool live = row < rows;
    const T* src = x + row * C;
    float v_[NV][E];
    float sum = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c0 = (sub + v * lpr) * E;
      const RawVec<16> raw = ldg_raw<16>(src + c0, live && c0 < C);
      widen(raw.r, v_[v], (const T*)nullptr);
#pragma unroll
      for (int e = 0; e < E; ++e) sum += v_[v][e];
    }
    for (int o = lpr >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum * inv_c;
    float sq = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c0 = (sub + v * lpr) * E;
      if (c0 < C) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float d = v_[v][e] - mean;
          sq = fmaf(d, d, sq);
        }
      }
    }
    for (int o = lpr >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq * inv_c + eps);
    if (live) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c0 = (sub + v * lpr) * E;
        if (c0 < C) {
          float o[E];
#pragma unroll
          for (int e = 0; e < E; ++e) {
            o[e] = fmaf((v_[v][e] - mean) * rstd, g[v][e], b[v][e]);
            if (GELU) o[e] = gelu_erf(to_f32(from_f32<T>(o[e])));
          }
          uint32_t packed[4];
          narrow(o, packed, (const T*)nullptr);
          stg_raw(y + row * C + c0, packed);
        }
      }
    }
  }
}

template <typename T, typename P>
static cudaError_t launch_tp(const T* x, const P* gamma, const P* beta, T* y, long long rows, int C, float eps,
                             int act, int sm_count, cudaStream_t s) {
  constexpr int E = 16 / (int)sizeof(T);
  const int n_vec = C / E;                       // C is a multiple of E (checked by the caller)
  int lpr = 1;
  while (lpr < 32 && lpr < n_vec) lpr *= 2;      // power of two >= min(n_vec, 32)
  if (lpr < 2) lpr = 2;
  const int nv = (n_vec + lpr - 1) / lpr;
  const int rows_per_warp = 32 / lpr;
  const long long warps_needed = (rows + rows_per_warp - 1) / rows_per_warp;
  long long blocks = (warps_needed + 7) / 8;
  const long long cap = (long long)sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
#define LN_CASE(NVV)                                                                                                   \
  case NVV:                                                                                                            \
    return act ? launch_overlapped(layernorm_fwd_kernel<T, P, NVV, true>, dim3((unsigned)blocks), dim3(256), 0, s, x,  \
                                   gamma, beta, y, rows, C, lpr, eps)                                                  \
               : launch_overlapped(layernorm_fwd_kernel<T, P, NVV, false>, dim3((unsigned)blocks), dim3(256), 0, s, x, \
                                   gamma, beta, y, rows, C, lpr, eps);
  switch (nv) {
    LN_CASE(1) LN_CASE(2) LN_CASE(3) LN_CASE(4) LN_CASE(5) LN_CASE(6) LN_CASE(7) LN_CASE(8)
    default: return cudaErrorInvalidValue;
  }
#undef LN_CASE
  return cudaGetLastError();
}

// dtype / param_dtype: 0 fp32, 1 fp16, 2 bf16; parameters are either fp32 or the tensor's own type.
// act: 0 none, 1 GELU (erf form) of the normalised value.
cudaError_t launch_layernorm_fwd(int dtype, int param_dtype, const void* x, const void* gamma, const void* beta,
                                 void* y, long long rows, int C, float eps, int act, int sm_count, cudaStream_t s) {
  const bool pf32 = param_dtype == 0;
  switch (dtype) {
    case 0:
      return launch_tp((const float*)x, (const float*)gamma, (const float*)beta, (float*)y, rows, C, eps, act, sm_count, s);
    case 1:
      return pf32 ? launch_tp((const __half*)x, (const float*)gamma, (const float*)beta, (__half*)y, rows, C, eps, act, sm_count, s)
                  : launch_tp((const __half*)x, (const __half*)gamma, (const __half*)beta, (__half*)y, rows, C, eps, act, sm_count, s);
    default:
      return pf32 ? launch_tp((const __nv_bfloat16*)x, (const float*)gamma, (const float*)beta, (__nv_bfloat16*)y, rows, C, eps, act, sm_count, s)
                  : launch_tp((const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta, (__nv_bfloat16*)y, rows, C, eps, act, sm_count, s);
  }
}

int layernorm_max_channels(int dtype) { return 32 * kLnMaxVec * (dtype == 0 ? 4 : 8); }

}  // namespace dcnb200
