// Shared device helpers for the DCNv4 / FlashDeformAttn kernels (sm_100a only).
//
// Conventions used by every kernel in this directory:
//  * tensors are channels-last; a "pair" is one (query, group) and owns D contiguous channels;
//  * forward: a lane owns a 32-byte channel vector of a pair (8 fp32 / 16 fp16-bf16 channels,
//    one 256-bit load per bilinear corner; 16 bytes when D is too small), so a 16-channel
//    fp16 group is one lane and the sampling arithmetic is not repeated per channel slice;
//  * backward: a lane owns 4 channels, so its grad_value contribution to a corner is exactly
//    one 16-byte vector reduction (red.global.add.v4.f32) and the lanes of a pair cover a
//    contiguous 64-byte (D=16) span per instruction;
//  * the lanes of a pair are adjacent, so offset/mask gradients are reduced with warp
//    shuffles and never with per-element atomics;
//  * a CTA owns a tile of queries whose packed offset/mask rows are staged into shared memory
//    with bulk asynchronous copies (TMA 1-D, no multicast) completed on one mbarrier;
//  * all arithmetic is fp32 whatever the storage type; results are rounded once on store.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dcnb200 {

constexpr int kThreads = 256;             // threads per CTA of the four main kernels
constexpr int kStageBytesMax = 40 * 1024; // shared-memory budget for one staged tile
constexpr int kMaxLevels = 8;             // FlashDeformAttn levels held in shared memory
constexpr int kMaxTileRows = 32;          // rows of a 2-D query tile (one bulk copy per row)

// Device status word values (written by a kernel that gave up on a bounded wait).
enum : int { kStatusOk = 0, kStatusStageTimeout = 1 };

// ----------------------------------------------------------------------------- storage types

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Predicated read-only gathers of BYTES = 8, 16 or 32 bytes; `ok == false` yields zeros
// (zero padding by omission).  The 32-byte form is a single 256-bit load
// (ld.global.nc.v8.b32, new with sm_100).
template <int BYTES> struct RawVec { uint32_t r[BYTES / 4]; };

template <int BYTES>
__device__ __forceinline__ RawVec<BYTES> ldg_raw(const void* p, bool ok);
template <>
__device__ __forceinline__ RawVec<8> ldg_raw<8>(const void* p, bool ok) {
  RawVec<8> v; v.r[0] = 0u; v.r[1] = 0u;
  if (ok) { const uint2 t = __ldg(reinterpret_cast<const uint2*>(p)); v.r[0] = t.x; v.r[1] = t.y; }
  return v;
}
template <>
__device__ __forceinline__ RawVec<16> ldg_raw<16>(const void* p, bool ok) {
  RawVec<16> v; v.r[0] = v.r[1] = v.r[2] = v.r[3] = 0u;
  if (ok) { const uint4 t = __ldg(reinterpret_cast<const uint4*>(p)); v.r[0] = t.x; v.r[1] = t.y; v.r[2] = t.z; v.r[3] = t.w; }
  return v;
}
template <>
__device__ __forceinline__ RawVec<32> ldg_raw<32>(const void* p, bool ok) {
  RawVec<32> v;
  asm("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %9, 0;\n\t"
      "mov.b32 %0, 0; mov.b32 %1, 0; mov.b32 %2, 0; mov.b32 %3, 0;\n\t"
      "mov.b32 %4, 0; mov.b32 %5, 0; mov.b32 %6, 0; mov.b32 %7, 0;\n\t"
      "@p ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n\t}"
      : "=r"(v.r[0]), "=r"(v.r[1]), "=r"(v.r[2]), "=r"(v.r[3]), "=r"(v.r[4]), "=r"(v.r[5]), "=r"(v.r[6]), "=r"(v.r[7])
      : "l"(p), "r"((int)ok));
  return v;
}

// raw storage words <-> fp32 channels (N channels of type T occupy N*sizeof(T)/4 words)
template <int N>
__device__ __forceinline__ void widen(const uint32_t (&r)[N], float (&v)[N], const float*) {
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = __uint_as_float(r[i]);
}
template <int N>
__device__ __forceinline__ void widen(const uint32_t (&r)[N / 2], float (&v)[N], const __half*) {
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&r[i]));
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
template <int N>
__device__ __forceinline__ void widen(const uint32_t (&r)[N / 2], float (&v)[N], const __nv_bfloat16*) {
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {  // bf16 -> fp32 is a 16-bit shift
    v[2 * i] = __uint_as_float(r[i] << 16);
    v[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
  }
}
template <int N>
__device__ __forceinline__ void narrow(const float (&v)[N], uint32_t (&r)[N], const float*) {
#pragma unroll
  for (int i = 0; i < N; ++i) r[i] = __float_as_uint(v[i]);
}
template <int N>
__device__ __forceinline__ void narrow(const float (&v)[N], uint32_t (&r)[N / 2], const __half*) {
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {
    const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    r[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
}
template <int N>
__device__ __forceinline__ void narrow(const float (&v)[N], uint32_t (&r)[N / 2], const __nv_bfloat16*) {
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    r[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
}
__device__ __forceinline__ void stg_raw(void* p, const uint32_t (&r)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void stg_raw(void* p, const uint32_t (&r)[4]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(r[0], r[1], r[2], r[3]);
}
__device__ __forceinline__ void stg_raw(void* p, const uint32_t (&r)[2]) {
  *reinterpret_cast<uint2*>(p) = make_uint2(r[0], r[1]);
}

// Vector reduction into an fp32 accumulation buffer (no return value -> RED, not ATOM).
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// ------------------------------------------------------------------- sampling coordinates

// DCNv4: base = p0 - c*s and coord = base + (tap*dil + offset)*s, each one fused
// multiply-add.  This operation order decides which pixels floor() selects and is shared
// with the corner-index probe kernels, so corner selection is reproducible bit for bit.
__device__ __forceinline__ float dcn_base(int p0, int c, float s) { return fmaf(-(float)c, s, (float)p0); }
__device__ __forceinline__ float dcn_coord(float base, float tap_dil, float off, float s) {
  return fmaf(tap_dil + off, s, base);
}
// FlashDeformAttn: round(loc*size) then subtract one half (two roundings, never fused).
__device__ __forceinline__ float fda_coord(float loc, float size) {
  return __fsub_rn(__fmul_rn(loc, size), 0.5f);
}
__device__ __forceinline__ bool in_range(float h, float w, float H, float W) {
  return h > -1.f && w > -1.f && h < H && w < W;
}

// Integral-valued float (|x| < 2^22) -> int without the conversion pipe: adding 1.5*2^23
// leaves the integer in the low mantissa bits.
__device__ __forceinline__ int int_of_integral(float x) {
  return __float_as_int(x + 12582912.f) - 0x4B400000;
}

// Bilinear footprint of a point (meaningful for in-range points only).
struct Footprint {
  int h0, w0;
  float lh, lw, hh, hw;
  bool top, bot, left, right;
};
__device__ __forceinline__ Footprint footprint(float h, float w, int H, int W) {
  Footprint f;
  const float hf = floorf(h), wf = floorf(w);
  f.h0 = int_of_integral(hf); f.w0 = int_of_integral(wf);
  f.lh = h - hf; f.lw = w - wf;
  f.hh = 1.f - f.lh; f.hw = 1.f - f.lw;
  f.top = f.h0 >= 0; f.bot = f.h0 < H - 1;
  f.left = f.w0 >= 0; f.right = f.w0 < W - 1;
  return f;
}

// One sampling point of the forward pass: gather the four corners of V = VB/sizeof(T)
// channels and accumulate m * bilinear.  `img` points at channel 0 of this lane in pixel (0,0).
template <typename T, int VB>
__device__ __forceinline__ void fwd_point(const T* __restrict__ img, int H, int W, int C, float h, float w,
                                          float m, float (&acc)[VB / (int)sizeof(T)]) {
  constexpr int V = VB / (int)sizeof(T);
  const bool ok = in_range(h, w, (float)H, (float)W);
  const Footprint f = footprint(h, w, H, W);
  const T* p1 = img + (ptrdiff_t)((f.h0 * W + f.w0) * C);
  const T* p3 = p1 + W * C;
  const RawVec<VB> r1 = ldg_raw<VB>(p1, ok && f.top && f.left);
  const RawVec<VB> r2 = ldg_raw<VB>(p1 + C, ok && f.top && f.right);
  const RawVec<VB> r3 = ldg_raw<VB>(p3, ok && f.bot && f.left);
  const RawVec<VB> r4 = ldg_raw<VB>(p3 + C, ok && f.bot && f.right);
  const float a = m * f.hh, b = m * f.lh;
  const float w1 = a * f.hw, w2 = a * f.lw, w3 = b * f.hw, w4 = b * f.lw;
  float v[V];
  widen(r1.r, v, (const T*)nullptr);
#pragma unroll
  for (int e = 0; e < V; ++e) acc[e] = fmaf(w1, v[e], acc[e]);
  widen(r2.r, v, (const T*)nullptr);
#pragma unroll
  for (int e = 0; e < V; ++e) acc[e] = fmaf(w2, v[e], acc[e]);
  widen(r3.r, v, (const T*)nullptr);
#pragma unroll
  for (int e = 0; e < V; ++e) acc[e] = fmaf(w3, v[e], acc[e]);
  widen(r4.r, v, (const T*)nullptr);
#pragma unroll
  for (int e = 0; e < V; ++e) acc[e] = fmaf(w4, v[e], acc[e]);
}

// One sampling point of the backward pass for a lane's 4 channels: scatter m*w_corner*gy into
// the fp32 accumulation buffer and return this lane's share of
//   gx = d(bilinear)/dw . gy,  gyv = d(bilinear)/dh . gy,  gm = bilinear . gy
// (added to the running values so several channel chunks can be summed before the shuffle).
// Returns whether the point passed the range test (false for inactive lanes).
template <typename T>
__device__ __forceinline__ bool bwd_point(const T* __restrict__ img, float* __restrict__ gimg, int H, int W,
                                          int C, float h, float w, float m, bool active, const float (&gy)[4],
                                          float& gx, float& gyv, float& gm) {
  constexpr int LB = 4 * (int)sizeof(T);
  const bool ok = active && in_range(h, w, (float)H, (float)W);
  const Footprint f = footprint(h, w, H, W);
  const ptrdiff_t pix = (ptrdiff_t)((f.h0 * W + f.w0) * C);
  const int row = W * C;
  const bool ok1 = ok && f.top && f.left, ok2 = ok && f.top && f.right;
  const bool ok3 = ok && f.bot && f.left, ok4 = ok && f.bot && f.right;
  const T* p1 = img + pix;
  const RawVec<LB> r1 = ldg_raw<LB>(p1, ok1);
  const RawVec<LB> r2 = ldg_raw<LB>(p1 + C, ok2);
  const RawVec<LB> r3 = ldg_raw<LB>(p1 + row, ok3);
  const RawVec<LB> r4 = ldg_raw<LB>(p1 + row + C, ok4);
  const float a = m * f.hh, b = m * f.lh;
  const float s1 = a * f.hw, s2 = a * f.lw, s3 = b * f.hw, s4 = b * f.lw;
  float* a1 = gimg + pix;
  if (ok1) red_add_v4(a1, s1 * gy[0], s1 * gy[1], s1 * gy[2], s1 * gy[3]);
  if (ok2) red_add_v4(a1 + C, s2 * gy[0], s2 * gy[1], s2 * gy[2], s2 * gy[3]);
  if (ok3) red_add_v4(a1 + row, s3 * gy[0], s3 * gy[1], s3 * gy[2], s3 * gy[3]);
  if (ok4) red_add_v4(a1 + row + C, s4 * gy[0], s4 * gy[1], s4 * gy[2], s4 * gy[3]);
  float v[4], d1, d2, d3, d4;
  widen(r1.r, v, (const T*)nullptr);
  d1 = fmaf(gy[0], v[0], fmaf(gy[1], v[1], fmaf(gy[2], v[2], gy[3] * v[3])));
  widen(r2.r, v, (const T*)nullptr);
  d2 = fmaf(gy[0], v[0], fmaf(gy[1], v[1], fmaf(gy[2], v[2], gy[3] * v[3])));
  widen(r3.r, v, (const T*)nullptr);
  d3 = fmaf(gy[0], v[0], fmaf(gy[1], v[1], fmaf(gy[2], v[2], gy[3] * v[3])));
  widen(r4.r, v, (const T*)nullptr);
  d4 = fmaf(gy[0], v[0], fmaf(gy[1], v[1], fmaf(gy[2], v[2], gy[3] * v[3])));
  gx += f.hh * (d2 - d1) + f.lh * (d4 - d3);
  gyv += f.hw * (d3 - d1) + f.lw * (d4 - d2);
  gm += f.hh * (f.hw * d1 + f.lw * d2) + f.lh * (f.hw * d3 + f.lw * d4);
  return ok;
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

// Stage `n_rows` spans of `row_bytes` each (global stride `src_stride` bytes, shared stride
// `dst_stride` bytes; every address and stride 16-byte aligned) into shared memory.  Whole
// 16-byte units go through bulk copies issued by thread 0 on one mbarrier; a ragged tail
// (< 16 bytes, only possible when n_rows == 1) is copied with plain loads.  Returns false on
// every thread of the CTA if the copies did not land within the bounded wait.
__device__ __forceinline__ bool stage_rows(void* smem_dst, const void* gsrc, uint32_t row_bytes, int n_rows,
                                           size_t src_stride, uint32_t dst_stride, uint64_t* bar, int* status) {
  const uint32_t bulk = row_bytes & ~15u;
  if (threadIdx.x == 0) mbar_init(bar, 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_expect_tx(bar, bulk * (uint32_t)n_rows);
    if (bulk)
      for (int r = 0; r < n_rows; ++r)
        bulk_g2s(static_cast<unsigned char*>(smem_dst) + (size_t)r * dst_stride,
                 static_cast<const unsigned char*>(gsrc) + (size_t)r * src_stride, bulk, bar);
  }
  if (threadIdx.x >= 32 && threadIdx.x < 32 + (row_bytes - bulk) / 2u) {  // tail, 2-byte granules
    const uint32_t i = bulk / 2u + (threadIdx.x - 32);
    reinterpret_cast<uint16_t*>(smem_dst)[i] = reinterpret_cast<const uint16_t*>(gsrc)[i];
  }
  bool landed = mbar_wait_bounded(bar, 0);
  if (!landed) {
    atomicExch(status, kStatusStageTimeout);
    mbar_wait_bounded(bar, 0);  // give the copies in flight one more bounded chance to finish
  }
  return __syncthreads_and(landed) != 0;
}

// --------------------------------------------------------------------------- parameters

struct DcnParams {
  int N, H, W, G, D, C, Ho, Wo;
  int kh, kw, sh, sw, ph, pw, dh, dw;
  int K, Ppad, remove_center, softmax;
  float scale;
  int th, tw;            // query tile (rows x columns) of one CTA
  int tiles_x, tiles_y;  // tiles per image
  int vb;                // forward: bytes of a lane's channel vector (16 or 32)
  int tpg, chunks;       // forward: D == (vb/elem) * tpg * chunks
  int tpg_b, chunks_b;   // backward: D == 4 * tpg_b * chunks_b
  int nq;                // N*Ho*Wo
};

struct FdaParams {
  int B, Len_in, G, D, C, L, Len_q, K, LK;
  int tile;              // consecutive queries per CTA
  int vb, tpg, chunks;   // forward lane geometry
  int tpg_b, chunks_b;   // backward lane geometry
  int nq;                // B*Len_q
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
