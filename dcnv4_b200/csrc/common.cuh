// Shared device helpers for the DCNv4 / FlashDeformAttn kernels (sm_100a only).
//
// Conventions used by every kernel in this directory:
//  * tensors are channels-last; a "pair" is one (query, group) and owns D contiguous channels;
//  * a thread owns a 16-byte channel vector (VEC = 4 fp32 / 8 fp16-bf16 channels) of a pair;
//    the `tpg` threads of a pair sit in consecutive lanes, so offset/mask gradients are
//    reduced with warp shuffles and never with per-element atomics;
//  * a CTA owns a tile of consecutive queries whose packed offset/mask rows form ONE
//    contiguous global span; that span is staged into shared memory with a single
//    bulk asynchronous copy (TMA, no multicast) completed on an mbarrier;
//  * all arithmetic is fp32 whatever the storage type; results are rounded once on store.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dcnb200 {

constexpr int kThreads = 256;            // threads per CTA of the four main kernels
constexpr int kStageBytesMax = 40 * 1024; // shared-memory budget for one staged tile
constexpr int kMaxLevels = 8;             // FlashDeformAttn levels held in shared memory

// Device status word values (written by a kernel that gave up on a bounded wait).
enum : int { kStatusOk = 0, kStatusStageTimeout = 1 };

// ----------------------------------------------------------------------------- storage types

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__half> { static constexpr int N = 8; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Unpack a 16-byte register quad into fp32 channel values.
__device__ __forceinline__ void unpack(const uint4& r, float (&v)[4], const float*) {
  v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y);
  v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
}
__device__ __forceinline__ void unpack(const uint4& r, float (&v)[8], const __half*) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void unpack(const uint4& r, float (&v)[8], const __nv_bfloat16*) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {  // bf16 -> fp32 is a 16-bit shift
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint4 pack(const float (&v)[4], const float*) {
  return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
}
__device__ __forceinline__ uint4 pack(const float (&v)[8], const __half*) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ uint4 pack(const float (&v)[8], const __nv_bfloat16*) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Read-only 16-byte gather of one channel vector; `ok == false` yields zeros (zero padding).
template <typename T>
__device__ __forceinline__ uint4 ldg_vec(const T* p, bool ok) {
  uint4 r = make_uint4(0u, 0u, 0u, 0u);
  if (ok) r = __ldg(reinterpret_cast<const uint4*>(p));
  return r;
}

// Vector reduction into an fp32 accumulation buffer (no return value -> RED, not ATOM).
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// ------------------------------------------------------------------- sampling coordinates

// DCNv4: base = p0 - c*s and coord = base + (tap*dil + offset)*s, each one fused
// multiply-add.  This operation order decides which pixels floor() selects and is shared
// with the corner-index debug kernels, so corner selection is reproducible bit for bit.
__device__ __forceinline__ float dcn_base(int p0, int c, float s) { return fmaf(-(float)c, s, (float)p0); }
__device__ __forceinline__ float dcn_coord(float base, int tap_dil, float off, float s) {
  return fmaf((float)tap_dil + off, s, base);
}
// FlashDeformAttn: round(loc*size) then subtract one half (two roundings, never fused).
__device__ __forceinline__ float fda_coord(float loc, int size) {
  return __fsub_rn(__fmul_rn(loc, (float)size), 0.5f);
}
__device__ __forceinline__ bool in_range(float h, float w, int H, int W) {
  return h > -1.f && w > -1.f && h < (float)H && w < (float)W;
}

// Bilinear footprint of an in-range point.
struct Footprint {
  int h0, w0;
  float lh, lw, hh, hw;
  bool top, bot, left, right;
};
__device__ __forceinline__ Footprint footprint(float h, float w, int H, int W) {
  Footprint f;
  const float hf = floorf(h), wf = floorf(w);
  f.h0 = (int)hf; f.w0 = (int)wf;
  f.lh = h - hf; f.lw = w - wf;
  f.hh = 1.f - f.lh; f.hw = 1.f - f.lw;
  f.top = f.h0 >= 0; f.bot = f.h0 + 1 < H;
  f.left = f.w0 >= 0; f.right = f.w0 + 1 < W;
  return f;
}

// ---------------------------------------------------------- mbarrier + bulk async copy (TMA)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: a staged copy normally lands within microseconds.  The limit only exists
// so that a lost copy can never hang the GPU; the caller then records an error and leaves.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < (1 << 22); ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// Stage `bytes` (element size `es` divides it) from a 16-byte aligned global address into
// 16-byte aligned shared memory.  Whole 16-byte units go through one bulk copy issued by
// thread 0; a ragged tail (< 16 bytes) is copied with plain loads.  Returns false on every
// thread of the CTA if the copy did not land within the bounded wait.
__device__ __forceinline__ bool stage_span(void* smem_dst, const void* gsrc, uint32_t bytes,
                                           uint64_t* bar, int* status) {
  const uint32_t bulk = bytes & ~15u;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_expect_tx(bar, bulk);
    if (bulk) bulk_g2s(smem_dst, gsrc, bulk, bar);
  }
  if (threadIdx.x >= 32 && threadIdx.x < 32 + (bytes - bulk) / 2u) {  // tail, 2-byte granules
    const uint32_t i = bulk / 2u + (threadIdx.x - 32);
    reinterpret_cast<uint16_t*>(smem_dst)[i] = reinterpret_cast<const uint16_t*>(gsrc)[i];
  }
  bool landed = mbar_wait_bounded(bar, 0);
  if (!landed) {
    atomicExch(status, kStatusStageTimeout);
    landed = mbar_wait_bounded(bar, 0);  // give the copy in flight one more bounded chance
    landed = false;
  }
  return __syncthreads_and(landed) != 0;
}

// --------------------------------------------------------------------------- parameters

struct DcnParams {
  int N, H, W, G, D, C, Ho, Wo;
  int kh, kw, sh, sw, ph, pw, dh, dw;
  int K, Ppad, remove_center, softmax;
  float scale;
  int tile;     // queries per CTA tile
  int tpg;      // threads per pair (power of two <= 32)
  int chunks;   // channel vectors per thread: D == VEC * tpg * chunks
  int nq;       // N*Ho*Wo
};

struct FdaParams {
  int B, Len_in, G, D, C, L, Len_q, K, LK;
  int tile, tpg, chunks;
  int nq;       // B*Len_q
};

// Host-side launchers (one per kernel family).  dtype: 0 fp32, 1 fp16, 2 bf16.
cudaError_t launch_dcnv4_fwd(int dtype, const void* value, const void* om, void* out,
                             const DcnParams& p, int* status, cudaStream_t s);
cudaError_t launch_dcnv4_bwd(int dtype, const void* value, const void* om, const void* gout,
                             float* gvalue_f32, void* gom, const DcnParams& p, int* status, cudaStream_t s);
cudaError_t launch_fda_fwd(int dtype, const void* value, const int64_t* shapes, const int64_t* starts,
                           const void* sla, void* out, const FdaParams& p, int* status, cudaStream_t s);
cudaError_t launch_fda_bwd(int dtype, const void* value, const int64_t* shapes, const int64_t* starts,
                           const void* sla, const void* gout, float* gvalue_f32, void* gsla,
                           const FdaParams& p, int* status, cudaStream_t s);
cudaError_t launch_convert_f32(int dtype, const float* src, void* dst, size_t n, cudaStream_t s);
cudaError_t launch_dcnv4_corners(int dtype, const void* om, int32_t* corners, const DcnParams& p, cudaStream_t s);
cudaError_t launch_fda_corners(int dtype, const int64_t* shapes, const void* sla, int32_t* corners,
                               const FdaParams& p, cudaStream_t s);

size_t dcnv4_fwd_smem(const DcnParams& p, int elem);
size_t dcnv4_bwd_smem(const DcnParams& p, int elem);
size_t fda_fwd_smem(const FdaParams& p, int elem);
size_t fda_bwd_smem(const FdaParams& p, int elem);

}  // namespace dcnb200
