// y = act(x + bias) over the last (contiguous) dimension of a channels-last 16-bit tensor.
//
// After BatchNorm folding the two stem convolutions of FlashInternImage carry a bias
// (classification/models/flash_intern_image.py:235-272: conv -> BN -> GELU -> conv -> BN).
// PyTorch runs a convolution bias as a separate broadcast `add_` and the GELU as another
// element-wise kernel over the largest activations of the network (N x 112 x 112 x 32); this
// kernel does both in one pass at memory speed.  GELU is evaluated by table (gelu_table.cuh),
// bit-identical to the erf formula on the rounded sum.
//
// Each thread owns one 16-byte column slot (8 channels) for the whole launch, so its bias is
// converted to fp32 once; the grid strides over rows of slots.
#include <mutex>

#include "common.cuh"
#include "gelu_table.cuh"

namespace dcnb200 {

namespace {

constexpr int kBiasActThreads = 512;

template <typename T, int ACT>
__global__ void __launch_bounds__(kBiasActThreads, ACT == 1 ? 1 : 2)
bias_act_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ y, long long n_vec, int cv,
                long long active_threads) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint16_t* lut = reinterpret_cast<uint16_t*>(smem_raw);
  if (ACT == 1) {
    gelu_lut_fill<T>(lut, threadIdx.x, kBiasActThreads);
    __syncthreads();
  }
  const long long tid = (long long)blockIdx.x * kBiasActThreads + threadIdx.x;
  pdl_trigger();
  pdl_wait();  // x is the previous kernel's output, and the bias may have been written by one (a fold, a cast)
  // `active_threads` is a multiple of the slots per row, so a thread's column never changes
  float b[8];
  {
    const int col = (int)(tid % cv) * 8;
    uint4 raw = __ldg(reinterpret_cast<const uint4*>(bias + col));
    const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = unpack2<T>(r[i]); b[2 * i] = f.x; b[2 * i + 1] = f.y; }
  }
  // Whole warps stay in the loop together (the table GELU votes across the warp): a lane past
  // the end works on a dummy vector and does not store.
  const long long warp_first = tid - (threadIdx.x & 31);
  for (long long i0 = warp_first; i0 < n_vec && warp_first < active_threads; i0 += active_threads) {
    const long long i = i0 + (threadIdx.x & 31);
    const bool live = tid < active_threads && i < n_vec;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (live) raw = *reinterpret_cast<const uint4*>(x + i * 8);
    const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = unpack2<T>(r[q]);
      o[q] = pack2<T>(f.x + b[2 * q], f.y + b[2 * q + 1]);  // rounded as the separate add would
    }
    if (ACT == 1) gelu_lut8<T>(o, lut);
    if (live) *reinterpret_cast<uint4*>(y + i * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <typename T, int ACT>
cudaError_t launch_act(const T* x, const T* bias, T* y, long long rows, int C, int sms, cudaStream_t s) {
  const size_t smem = ACT == 1 ? (size_t)gelu_lut_bytes<T>() : 0;
  if (ACT == 1) {
    static std::once_flag once[64];
    static cudaError_t err[64];
    int dev = 0;
    cudaGetDevice(&dev);
    dev = dev < 0 || dev >= 64 ? 0 : dev;
    std::call_once(once[dev], [&] {
      err[dev] = cudaFuncSetAttribute(bias_act_kernel<T, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    });
    if (err[dev] != cudaSuccess) return err[dev];
  }
  const int cv = C / 8;
  const long long n_vec = rows * cv;
  long long blocks = (long long)sms * (ACT == 1 ? 1 : 2) * 2;  // a few waves of persistent-ish CTAs
  const long long need = (n_vec + kBiasActThreads - 1) / kBiasActThreads;
  if (blocks > need) blocks = need;
  if (blocks < 1) blocks = 1;
  long long active = blocks * kBiasActThreads / cv * cv;  // largest multiple of the row's slot count
  if (active < cv) {  // rows wider than the whole grid: grow the grid to one row of slots
    blocks = (cv + kBiasActThreads - 1) / kBiasActThreads;
    active = blocks * kBiasActThreads / cv * cv;
  }
  return launch_overlapped(bias_act_kernel<T, ACT>, dim3((unsigned)blocks), dim3(kBiasActThreads), smem, s, x, bias, y,
                           n_vec, cv, active);
}

}  // namespace

// dtype 1 fp16 / 2 bf16; act 0 none / 1 GELU.  C a multiple of 8; y may alias x.
cudaError_t launch_bias_act_fwd(int dtype, const void* x, const void* bias, void* y, long long rows, int C, int act,
                                int sms, cudaStream_t s) {
  if (dtype == 1) {
    using T = __half;
    return act ? launch_act<T, 1>((const T*)x, (const T*)bias, (T*)y, rows, C, sms, s)
               : launch_act<T, 0>((const T*)x, (const T*)bias, (T*)y, rows, C, sms, s);
  }
  using T = __nv_bfloat16;
  return act ? launch_act<T, 1>((const T*)x, (const T*)bias, (T*)y, rows, C, sms, s)
             : launch_act<T, 0>((const T*)x, (const T*)bias, (T*)y, rows, C, sms, s);
}

}  // namespace dcnb200
