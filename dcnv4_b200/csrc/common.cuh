// Shared device helpers for the DCNv4 / FlashDeformAttn kernels (sm_100a only).
//
// Conventions used by every kernel in this directory:
//  * tensors are channels-last; a "pair" is one (query, group) and owns D contiguous channels;
//  * forward: a lane owns 32 bytes of a pair's channels (a whole 16-channel fp16/bf16 group,
//    half of an fp32 one; 16 bytes when size or alignment forbid) and fetches a bilinear
//    corner with one 256-bit load, so the lanes of a pair cover the corner in ONE instruction;
//  * backward: a lane owns 4 channels: exactly one 16-byte vector reduction
//    (red.global.add.v4.f32) per corner into the fp32 accumulation buffer, the lanes of a pair
//    again covering the corner's contiguous bytes in one instruction.  (The kernels are
//    templates on the channels per lane; api.cu:lane_geometry picks these values from measured
//    gather / reduction rates.);
//  * the lanes of a pair are adjacent, so offset/mask gradients are reduced with warp
//    shuffles and never with per-element atomics;
//  * CTAs are persistent: each loops over query tiles, and while it works on one tile the
//    packed offset/mask rows of its next tile are already in flight into the other half of a
//    double-buffered shared-memory stage (bulk asynchronous copies, TMA 1-D, no multicast,
//    one mbarrier per buffer, bounded waits);
//  * all arithmetic is fp32 whatever the storage type; results are rounded once on store.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

namespace dcnb200 {

// Resident CTAs per SM the kernels are compiled for (bounds the registers per thread).
#ifndef DCNB200_FWD_MINB
#define DCNB200_FWD_MINB 2
#endif
#ifndef DCNB200_BWD_MINB
#define DCNB200_BWD_MINB 3
#endif

constexpr int kThreads = 256;             // threads per CTA of the four main kernels
constexpr int kSmemBudget = 72 * 1024;    // dynamic shared memory one CTA may use (3 CTAs per SM fit)
constexpr int kMaxLevels = 8;             // FlashDeformAttn levels held in shared memory
constexpr int kMaxTileRows = 32;          // rows of a 2-D query tile (one bulk copy per row)

// Device status word values (written by a kernel that gave up on a bounded wait).
enum : int {
  kStatusOk = 0,
  kStatusStageTimeout = 1,  // a staged copy never landed within the bounded wait
  kStatusBadLevels = 2      // a FlashDeformAttn level does not lie inside the flattened value tensor
};

// FlashDeformAttn level table entry (H, W, first row) from the two int64 device tensors, checked
// against the flattened length: a level that starts before 0 or ends after Len_in -- a caller-side
// bug, stale shapes, (W,H) order with the wrong starts -- is replaced by an empty level (H = W = 0,
// every sample then fails the range test and contributes nothing) and recorded in the status
// word, so that neither the gathers nor the gradient reductions can leave the tensors.
__device__ __forceinline__ void load_level(int* dst, const int64_t* shapes, const int64_t* starts, int l,
                                           int len_in, int* status) {
  const long long H = shapes[2 * l], W = shapes[2 * l + 1], s0 = starts[l];
  const bool ok = H >= 0 && W >= 0 && s0 >= 0 && H <= len_in && W <= len_in && H * W <= (long long)len_in - s0;
  dst[0] = ok ? (int)H : 0;
  dst[1] = ok ? (int)W : 0;
  dst[2] = ok ? (int)s0 : 0;
  if (!ok) atomicExch(status, kStatusBadLevels);
}

// ----------------------------------------------------------------------------- storage types

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 32 bytes of zeros.  A bilinear corner that lies outside the map is read from here instead
// of being predicated off: the load stays unconditional (no per-register zero fill, no
// predicate) and the out-of-map corner still contributes exactly zero.
static __device__ __align__(32) const uint32_t g_zero_page[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};

// Read-only gathers of BYTES = 8, 16 or 32 bytes; `ok == false` reads the zero page (zero
// padding).  The 32-byte form is a single 256-bit load (ld.global.nc.v8.b32, new with sm_100).
template <int BYTES> struct RawVec { uint32_t r[BYTES / 4]; };

template <int BYTES>
__device__ __forceinline__ RawVec<BYTES> ldg_raw(const void* p, bool ok);
template <>
__device__ __forceinline__ RawVec<8> ldg_raw<8>(const void* p, bool ok) {
  const uint2 t = __ldg(reinterpret_cast<const uint2*>(ok ? p : (const void*)g_zero_page));
  RawVec<8> v; v.r[0] = t.x; v.r[1] = t.y;
  return v;
}
template <>
__device__ __forceinline__ RawVec<16> ldg_raw<16>(const void* p, bool ok) {
  const uint4 t = __ldg(reinterpret_cast<const uint4*>(ok ? p : (const void*)g_zero_page));
  RawVec<16> v; v.r[0] = t.x; v.r[1] = t.y; v.r[2] = t.z; v.r[3] = t.w;
  return v;
}
template <>
__device__ __forceinline__ RawVec<32> ldg_raw<32>(const void* p, bool ok) {
  RawVec<32> v;
  const void* q = ok ? p : (const void*)g_zero_page;
  asm("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(v.r[0]), "=r"(v.r[1]), "=r"(v.r[2]), "=r"(v.r[3]), "=r"(v.r[4]), "=r"(v.r[5]), "=r"(v.r[6]), "=r"(v.r[7])
      : "l"(q));
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
// FlashDeformAttn: loc*size - 0.5 as ONE fused multiply-add, which is what the reference
// binary does (verified against its kernels on a B200 at samples whose product lands on x.5).
__device__ __forceinline__ float fda_coord(float loc, float size) {
  return fmaf(loc, size, -0.5f);
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

// Gather V channels (V*sizeof(T) = 16, 32 or 64 bytes; 64 bytes = two 256-bit loads) of one
// bilinear corner as fp32.
template <typename T, int V>
__device__ __forceinline__ void gather_corner(const T* p, bool ok, float (&v)[V]) {
  constexpr int B = V * (int)sizeof(T);
  if constexpr (B == 64) {
    const RawVec<32> a = ldg_raw<32>(p, ok);
    const RawVec<32> b = ldg_raw<32>(p + V / 2, ok);
    float lo[V / 2], hi[V / 2];
    widen(a.r, lo, (const T*)nullptr);
    widen(b.r, hi, (const T*)nullptr);
#pragma unroll
    for (int e = 0; e < V / 2; ++e) { v[e] = lo[e]; v[V / 2 + e] = hi[e]; }
  } else {
    const RawVec<B> a = ldg_raw<B>(p, ok);
    widen(a.r, v, (const T*)nullptr);
  }
}

// One sampling point of the forward pass: gather the four corners of this lane's V channels
// and accumulate m * bilinear.  `img` points at channel 0 of this lane in pixel (0,0).
template <typename T, int V>
__device__ __forceinline__ void fwd_point(const T* __restrict__ img, int H, int W, int C, float Hf, float Wf,
                                          float h, float w, float m, float (&acc)[V]) {
  const bool ok = in_range(h, w, Hf, Wf);
  const Footprint f = footprint(h, w, H, W);
  const int row = W * C;
  const int i1 = (f.h0 * W + f.w0) * C;
  float v1[V], v2[V], v3[V], v4[V];
  gather_corner<T, V>(img + i1, ok && f.top && f.left, v1);
  gather_corner<T, V>(img + (i1 + C), ok && f.top && f.right, v2);
  gather_corner<T, V>(img + (i1 + row), ok && f.bot && f.left, v3);
  gather_corner<T, V>(img + (i1 + row + C), ok && f.bot && f.right, v4);
  const float a = m * f.hh, b = m * f.lh;
  const float w1 = a * f.hw, w2 = a * f.lw, w3 = b * f.hw, w4 = b * f.lw;
#pragma unroll
  for (int e = 0; e < V; ++e)
    acc[e] = fmaf(w1, v1[e], fmaf(w2, v2[e], fmaf(w3, v3[e], fmaf(w4, v4[e], acc[e]))));
}

// One sampling point of the backward pass for a lane's V channels (V = 4 or 8): scatter
// m*w_corner*gy into the fp32 accumulation buffer with 16-byte vector reductions and add this
// lane's share of
//   gx = d(bilinear)/dw . gy,  gyv = d(bilinear)/dh . gy,  gm = bilinear . gy
// to the running values (so several channel chunks can be summed before the shuffle).
// Returns whether the point passed the range test (false for inactive lanes).
template <typename T, int V>
__device__ __forceinline__ bool bwd_point(const T* __restrict__ img, float* __restrict__ gimg, int H, int W,
                                          int C, float Hf, float Wf, float h, float w, float m, bool active,
                                          const float (&gy)[V], float& gx, float& gyv, float& gm) {
  const bool ok = active && in_range(h, w, Hf, Wf);
  const Footprint f = footprint(h, w, H, W);
  const int row = W * C;
  const int i1 = (f.h0 * W + f.w0) * C;
  const bool ok1 = ok && f.top && f.left, ok2 = ok && f.top && f.right;
  const bool ok3 = ok && f.bot && f.left, ok4 = ok && f.bot && f.right;
  float v1[V], v2[V], v3[V], v4[V];
  gather_corner<T, V>(img + i1, ok1, v1);
  gather_corner<T, V>(img + (i1 + C), ok2, v2);
  gather_corner<T, V>(img + (i1 + row), ok3, v3);
  gather_corner<T, V>(img + (i1 + row + C), ok4, v4);
  const float a = m * f.hh, b = m * f.lh;
  const float s1 = a * f.hw, s2 = a * f.lw, s3 = b * f.hw, s4 = b * f.lw;
#pragma unroll
  for (int e = 0; e < V; e += 4) {
    if (ok1) red_add_v4(gimg + (i1 + e), s1 * gy[e], s1 * gy[e + 1], s1 * gy[e + 2], s1 * gy[e + 3]);
    if (ok2) red_add_v4(gimg + (i1 + C + e), s2 * gy[e], s2 * gy[e + 1], s2 * gy[e + 2], s2 * gy[e + 3]);
    if (ok3) red_add_v4(gimg + (i1 + row + e), s3 * gy[e], s3 * gy[e + 1], s3 * gy[e + 2], s3 * gy[e + 3]);
    if (ok4) red_add_v4(gimg + (i1 + row + C + e), s4 * gy[e], s4 * gy[e + 1], s4 * gy[e + 2], s4 * gy[e + 3]);
  }
  float d1 = 0.f, d2 = 0.f, d3 = 0.f, d4 = 0.f;  // sum_c gy_c * v_corner,c
#pragma unroll
  for (int e = 0; e < V; ++e) {
    d1 = fmaf(gy[e], v1[e], d1);
    d2 = fmaf(gy[e], v2[e], d2);
    d3 = fmaf(gy[e], v3[e], d3);
    d4 = fmaf(gy[e], v4[e], d4);
  }
  gx += f.hh * (d2 - d1) + f.lh * (d4 - d3);
  gyv += f.hw * (d3 - d1) + f.lw * (d4 - d2);
  gm += f.hh * (f.hw * d1 + f.lw * d2) + f.lh * (f.hw * d3 + f.lw * d4);
  return ok;
}

// Division of a small non-negative int by a runtime constant without the integer-divide
// sequence: q = umulhi(n, mul) with mul = floor(2^32/d) + 1 is exact while n*d < 2^32
// (tile-local indices are a few thousand at most); d == 1 is passed through.
struct FastDiv { uint32_t d, mul; };
__device__ __forceinline__ int fast_div(int n, const FastDiv& f) {
  return f.d == 1 ? n : (int)__umulhi((uint32_t)n, f.mul);
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

// Issue (thread 0 only) the bulk copies of one staged tile: `n_rows` spans of `row_bytes`
// each (global stride `src_stride` bytes, shared stride `dst_stride` bytes; every address and
// stride 16-byte aligned), all completing on `bar`.  Only whole 16-byte units are copied; a
// ragged tail (< 16 bytes, only possible when n_rows == 1) is left to copy_tail().
__device__ __forceinline__ void issue_stage(void* smem_dst, const void* gsrc, uint32_t row_bytes, int n_rows,
                                            size_t src_stride, uint32_t dst_stride, uint64_t* bar) {
  const uint32_t bulk = row_bytes & ~15u;
  mbar_expect_tx(bar, bulk * (uint32_t)n_rows);
  if (bulk)
    for (int r = 0; r < n_rows; ++r)
      bulk_g2s(static_cast<unsigned char*>(smem_dst) + (size_t)r * dst_stride,
               static_cast<const unsigned char*>(gsrc) + (size_t)r * src_stride, bulk, bar);
}
// Ragged tail of a single-span stage, copied with plain 2-byte loads by a few threads.
__device__ __forceinline__ void copy_tail(void* smem_dst, const void* gsrc, uint32_t row_bytes) {
  const uint32_t bulk = row_bytes & ~15u;
  if (threadIdx.x < (row_bytes - bulk) / 2u) {
    const uint32_t i = bulk / 2u + threadIdx.x;
    reinterpret_cast<uint16_t*>(smem_dst)[i] = reinterpret_cast<const uint16_t*>(gsrc)[i];
  }
}
// Wait (bounded) for a staged tile.  A copy that never lands is recorded in the status word
// and the CTA carries on: every gather and scatter is range-checked, so stale staging data
// can produce wrong numbers but never an out-of-bounds access or a hang.
__device__ __forceinline__ void wait_stage(uint64_t* bar, uint32_t parity, int* status) {
  if (!mbar_wait_bounded(bar, parity)) atomicExch(status, kStatusStageTimeout);
}

// ------------------------------------------------------ programmatic dependent launch
//
// The inference-path kernels (LayerNorm, Linear, DCNv4 forward) are launched so that their
// prologue -- barrier set-up, tensor-memory allocation, table fill -- may start while the
// previous kernel of the stream is still draining.  pdl_wait() blocks until that kernel has
// completed and its writes are visible; it must precede the first access to global memory that
// another kernel may have written and every write to global memory.  pdl_trigger() lets the
// next kernel's prologue start.  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#ifndef DCNB200_PDL
#define DCNB200_PDL 1
#endif
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped_if(bool allow, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // DCNV4B200_PDL=0 in the environment (read once) launches every kernel the ordinary way: an aid for
  // telling apart a kernel's own time from what the overlap with its neighbours adds or hides.
  static const bool enabled = [] { const char* v = getenv("DCNV4B200_PDL"); return !(v && v[0] == '0'); }();
  cfg.numAttrs = (DCNB200_PDL && enabled && allow) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                              Args&&... args) {
  return launch_overlapped_if(true, kern, grid, block, smem, s, static_cast<Args&&>(args)...);
}
// Shared-memory carve-out hint for a kernel that lives on L1 hits.  A kernel launched with programmatic
// stream serialization inherits the L1 / shared-memory split of the kernel before it unless it states
// a preference of its own: behind a tensor-core Linear (220 KB of shared memory per SM, 28 KB of L1
// left) the DCNv4 forward ran 30-100 % slower (measured at batch 256: 56x56x64 sequence 461 instead of
// 340 us, 14x14x256 200 instead of 112 us).  `bytes_per_sm` is what the kernel's resident CTAs need;
// the hint is the smallest percentage of the 228 KB that covers it, set once per value and device.
template <auto Kern>
inline void prefer_carveout(size_t bytes_per_sm) {
  static int current[64] = {0};  // per kernel (template argument) and device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  dev &= 63;
  int pct = (int)((bytes_per_sm * 100 + 228 * 1024 - 1) / (228 * 1024));
  pct = pct < 1 ? 1 : (pct > 100 ? 100 : pct);
  if (current[dev] == pct) return;
  if (cudaFuncSetAttribute(Kern, cudaFuncAttributePreferredSharedMemoryCarveout, pct) == cudaSuccess) current[dev] = pct;
}

// --------------------------------------------------------------------------- parameters

struct DcnParams {
  int N, H, W, G, D, C, Ho, Wo;
  int kh, kw, sh, sw, ph, pw, dh, dw;
  int K, Ppad, remove_center, softmax;
  float scale;
  int th, tw;            // query tile (rows x columns) of one CTA
  int tiles_x, tiles_y;  // tiles per image
  int lane_ch, tpg, chunks;        // forward: D == lane_ch * tpg * chunks
  int lane_ch_b, tpg_b, chunks_b;  // backward: D == lane_ch_b * tpg_b * chunks_b
  int nq;                // N*Ho*Wo
  int sm_count;          // SMs of the current device (persistent grid sizing)
  FastDiv div_g, div_tw;
};

struct FdaParams {
  int B, Len_in, G, D, C, L, Len_q, K, LK;
  int tile;              // consecutive queries per CTA
  int lane_ch, tpg, chunks;        // forward lane geometry
  int lane_ch_b, tpg_b, chunks_b;  // backward lane geometry
  int nq;                // B*Len_q
  int sm_count;
  FastDiv div_g;
};

// Host-side launchers (one per kernel family).  dtype: 0 fp32, 1 fp16, 2 bf16.
cudaError_t launch_dcnv4_fwd(int dtype, const void* value, const void* om, void* out,
                             const DcnParams& p, int* status, cudaStream_t s);
cudaError_t launch_dcnv4_bwd(int dtype, const void* value, const void* om, const void* gout,
                             float* gvalue_f32, void* gom, const DcnParams& p, int* status, cudaStream_t s);
// Spatially tiled variants (value tile and, for the backward, the grad_value tile in shared
// memory; dcnv4_*_tiled.cu).  `*_applies` says whether the configuration is covered.
bool dcnv4_fwd_tiled_applies(const DcnParams& p);
cudaError_t launch_dcnv4_fwd_tiled(int dtype, const void* value, const void* om, void* out, const DcnParams& p,
                                   int* status, cudaStream_t s);
bool dcnv4_bwd_tiled_applies(const DcnParams& p);
cudaError_t launch_dcnv4_bwd_tiled(int dtype, const void* value, const void* om, const void* gout,
                                   float* gvalue_f32, void* gom, const DcnParams& p, int* status, cudaStream_t s);
// DCNv4 forward that computes its offset/mask rows itself from the layer input and the weights of the
// module's offset/mask Linear (dcnv4_fwd_fused.cu; 16-bit tensors, 3x3 / stride 1 / pad 1 /
// dilation 1, D = 16).
bool dcnv4_fwd_fused_applies(int dtype, int G, int D, int K, int w_rows);
cudaError_t launch_dcnv4_fwd_fused(int dtype, const void* value, const void* x, const void* w, const void* bias,
                                   void* out, int N, int H, int W, int G, int K, int w_rows, float scale, int sms,
                                   int* status, cudaStream_t stream);
// Kernel choice for configurations both kernels cover: environment variable DCNV4B200_TILED,
// read at every call; 1 selects the tiled kernel, anything else (-1 unset, 0) the default one.
// Meant for A/B measurements and for the tests of the tiled kernel.
int tiled_override();
cudaError_t launch_fda_fwd(int dtype, const void* value, const int64_t* shapes, const int64_t* starts,
                           const void* sla, void* out, const FdaParams& p, int* status, cudaStream_t s);
cudaError_t launch_fda_bwd(int dtype, const void* value, const int64_t* shapes, const int64_t* starts,
                           const void* sla, const void* gout, float* gvalue_f32, void* gsla,
                           const FdaParams& p, int* status, cudaStream_t s);
cudaError_t launch_convert_f32(int dtype, const float* src, void* dst, size_t n, int sm_count, cudaStream_t s);
cudaError_t launch_dcnv4_corners(int dtype, const void* om, int32_t* corners, const DcnParams& p, cudaStream_t s);
cudaError_t launch_fda_corners(int dtype, const int64_t* shapes, const void* sla, int32_t* corners,
                               const FdaParams& p, cudaStream_t s);

// Resident CTAs per SM of a persistent kernel, without a runtime query per launch.  The first
// launch of each kernel on each device raises its dynamic shared-memory limit to the budget
// and reads its register count; afterwards the answer is arithmetic on the launch's
// shared-memory size.  An over-estimate is harmless: CTAs never wait on one another, a CTA
// that is not resident at once simply starts when a slot frees up.
template <auto Kern>
inline cudaError_t persistent_ctas_per_sm(size_t smem, int* per_sm) {
  static int regs_limit[64] = {0};  // per device; written once with the same value by any thread
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  dev &= 63;
  int lim = regs_limit[dev];
  if (lim == 0) {
    e = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e != cudaSuccess) return e;
    cudaFuncAttributes a;
    e = cudaFuncGetAttributes(&a, Kern);
    if (e != cudaSuccess) return e;
    const int regs_per_cta = ((a.numRegs + 7) / 8 * 8) * kThreads;
    lim = regs_per_cta > 0 ? 65536 / regs_per_cta : 1;
    if (lim < 1) lim = 1;
    regs_limit[dev] = lim;
  }
  int by_smem = (int)((227u * 1024u) / (smem + 1024u));
  int n = lim < by_smem ? lim : by_smem;
  if (n > 2048 / kThreads) n = 2048 / kThreads;
  *per_sm = n < 1 ? 1 : n;
  return cudaSuccess;
}

cudaError_t launch_layernorm_fwd(int dtype, int param_dtype, const void* x, const void* gamma, const void* beta,
                                 void* y, long long rows, int C, float eps, int act, int sm_count, cudaStream_t s);
int layernorm_max_channels(int dtype);

// out = x*(1 - s) + x_proj*s with s = sigmoid(x . weight^T + bias) per row and group (center_scale.cu).
cudaError_t launch_center_scale_blend(int dtype, int param_dtype, const void* x, const void* xp, const void* w,
                                      const void* b, void* out, long long rows, int G, int D, int sm_count,
                                      cudaStream_t s);
int center_scale_max_channels(int dtype);
int center_scale_max_groups();

// y = epilogue(x . W^T + bias) on the tensor cores (linear.cu); dtype 1 fp16 / 2 bf16.
cudaError_t launch_linear_fwd(int dtype, const void* x, const void* w, const void* bias, const void* residual,
                              void* y, long long M, int N, int K, int act, int sms, int* status,
                              cudaStream_t stream, const void* gamma = nullptr, const void* beta = nullptr,
                              float eps = 0.f, void* z = nullptr, int n_split = 0);

// y = act(x + bias) over the channels of a channels-last 16-bit tensor (bias_act.cu).
cudaError_t launch_bias_act_fwd(int dtype, const void* x, const void* bias, void* y, long long rows, int C, int act,
                                int sms, cudaStream_t s);

size_t dcnv4_fwd_smem(const DcnParams& p, int elem);
size_t dcnv4_bwd_smem(const DcnParams& p, int elem);
size_t fda_fwd_smem(const FdaParams& p, int elem);
size_t fda_bwd_smem(const FdaParams& p, int elem);

}  // namespace dcnb200
