// Small companion kernels: the fp32 -> fp16/bf16 finalize of the backward accumulation
// buffer (the fused replacement of the reference's `.to(kHalf)` pass,
// DCNv4_op/src/cuda/dcnv4_cuda.cu:169-171) and the corner-index probes used by the parity
// tests to check that floor() of the sampling coordinates selects the same pixels as the
// reference formula (DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:203-224,
// DCNv4_op/src/cuda/flash_deform_im2col_cuda.cuh:185-190, DCNv4_op/src/cuda/common.h:47-48).
#include "common.cuh"

namespace dcnb200 {

constexpr int kSkipped = INT32_MIN;

template <typename T>
__global__ void convert_kernel(const float4* __restrict__ src, T* __restrict__ dst, size_t n8, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const float4 a = src[2 * i], b = src[2 * i + 1];
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t packed[4];
    narrow(v, packed, (const T*)nullptr);
    stg_raw(dst + i * 8, packed);
  }
  // ragged tail (n not a multiple of 8)
  if (blockIdx.x == 0) {
    const float* s = reinterpret_cast<const float*>(src);
    for (size_t i = n8 * 8 + threadIdx.x; i < n; i += blockDim.x) dst[i] = from_f32<T>(s[i]);
  }
}

cudaError_t launch_convert_f32(int dtype, const float* src, void* dst, size_t n, int sm_count, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const size_t n8 = n / 8;
  const int block = 256;
  size_t want = (n8 + block - 1) / block;
  const size_t cap = (size_t)(sm_count > 0 ? sm_count : 1) * 16;
  const int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
  if (dtype == 1)
    convert_kernel<__half><<<grid, block, 0, s>>>((const float4*)src, (__half*)dst, n8, n);
  else
    convert_kernel<__nv_bfloat16><<<grid, block, 0, s>>>((const float4*)src, (__nv_bfloat16*)dst, n8, n);
  return cudaGetLastError();
}

template <typename T>
__global__ void dcnv4_corners_kernel(const T* __restrict__ om, int32_t* __restrict__ corners, const DcnParams p) {
  const size_t total = (size_t)p.nq * p.G * p.K;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int k = (int)(i % p.K);
  const int g = (int)((i / p.K) % p.G);
  const int q = (int)(i / ((size_t)p.K * p.G));
  const int rem = q % (p.Ho * p.Wo);
  const int y = rem / p.Wo, x = rem % p.Wo;
  const int center = (p.kw / 2) * p.kh + (p.kh / 2);
  const int t = k + ((p.remove_center && k >= center) ? 1 : 0);  // tap index of point k
  const int ti = t / p.kh, tj = t % p.kh;
  const int cw = (p.dw * (p.kw - 1)) >> 1, ch = (p.dh * (p.kh - 1)) >> 1;
  const T* row = om + (size_t)q * p.Ppad + g * 3 * p.K;
  const float w_im = dcn_coord(dcn_base(cw - p.pw + x * p.sw, cw, p.scale), (float)(ti * p.dw), to_f32(row[2 * k]), p.scale);
  const float h_im = dcn_coord(dcn_base(ch - p.ph + y * p.sh, ch, p.scale), (float)(tj * p.dh), to_f32(row[2 * k + 1]), p.scale);
  int h0 = kSkipped, w0 = kSkipped;
  if (in_range(h_im, w_im, (float)p.H, (float)p.W)) {
    const Footprint f = footprint(h_im, w_im, p.H, p.W);
    h0 = f.h0; w0 = f.w0;
  }
  corners[2 * i] = h0;
  corners[2 * i + 1] = w0;
}

cudaError_t launch_dcnv4_corners(int dtype, const void* om, int32_t* corners, const DcnParams& p, cudaStream_t s) {
  const size_t total = (size_t)p.nq * p.G * p.K;
  const int grid = (int)((total + 255) / 256);
  if (dtype == 0) dcnv4_corners_kernel<float><<<grid, 256, 0, s>>>((const float*)om, corners, p);
  else if (dtype == 1) dcnv4_corners_kernel<__half><<<grid, 256, 0, s>>>((const __half*)om, corners, p);
  else dcnv4_corners_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)om, corners, p);
  return cudaGetLastError();
}

template <typename T>
__global__ void fda_corners_kernel(const int64_t* __restrict__ shapes, const T* __restrict__ sla,
                                   int32_t* __restrict__ corners, const FdaParams p) {
  const size_t total = (size_t)p.nq * p.G * p.LK;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int t = (int)(i % p.LK);
  const size_t pr = i / p.LK;
  const int l = t / p.K;
  const int Hl = (int)shapes[2 * l], Wl = (int)shapes[2 * l + 1];
  const T* row = sla + pr * 3 * p.LK;
  const float w_im = fda_coord(to_f32(row[2 * t]), (float)Wl);
  const float h_im = fda_coord(to_f32(row[2 * t + 1]), (float)Hl);
  int h0 = kSkipped, w0 = kSkipped;
  if (in_range(h_im, w_im, (float)Hl, (float)Wl)) {
    const Footprint f = footprint(h_im, w_im, Hl, Wl);
    h0 = f.h0; w0 = f.w0;
  }
  corners[2 * i] = h0;
  corners[2 * i + 1] = w0;
}

cudaError_t launch_fda_corners(int dtype, const int64_t* shapes, const void* sla, int32_t* corners,
                               const FdaParams& p, cudaStream_t s) {
  const size_t total = (size_t)p.nq * p.G * p.LK;
  const int grid = (int)((total + 255) / 256);
  if (dtype == 0) fda_corners_kernel<float><<<grid, 256, 0, s>>>(shapes, (const float*)sla, corners, p);
  else if (dtype == 1) fda_corners_kernel<__half><<<grid, 256, 0, s>>>(shapes, (const __half*)sla, corners, p);
  else fda_corners_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(shapes, (const __nv_bfloat16*)sla, corners, p);
  return cudaGetLastError();
}

}  // namespace dcnb200
