// DCNv4 forward with the spatial tile of `value` staged in shared memory.
//
// Replaces, for the configuration every FlashInternImage layer uses (3x3, stride 1, dilation 1,
// 16 channels per group, a multiple of four groups, no softmax, centre kept), the same reference
// code as dcnv4_fwd.cu: forward_kernel_dcn_reg and its launcher
// (DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:142-325), whose every bilinear corner is a global
// load (common.h:74-90).  Every other configuration keeps the kernel of dcnv4_fwd.cu.
//
// A CTA (8 warps) works on a task = 8x8 output positions x 4 groups:
//  * the pixel box those positions can sample from (tile + 4-pixel halo) is brought into shared
//    memory by four tiled TMA loads, one per group (cp.async.bulk.tensor.4d over this GPU's own
//    memory, no multicast; pixels outside the image arrive as zeros = the operator's zero
//    padding), each box group-major [row][column][16 channels];
//  * a warp owns one row of the tile: 8 positions x 4 groups = 32 (position, group) pairs.  For one
//    kernel tap at a time, lane l prepares the sampling point of pair l once -- corner offset in
//    the box and the four bilinear weights times the mask -- and leaves it in a small per-warp
//    record buffer (the offset/mask values of the next tap are already on their way from global
//    memory while the current tap is processed);
//  * the quarter-warps then take the 32 points four at a time, a quarter-warp per point:
//      fp32: lanes 0-3 read the four channel quads of the top-left corner and lanes 4-7 those of
//            the top-right one, which the group-major layout puts next to each other: one 128-bit
//            load per lane covers a contiguous 128-byte span = every bank once, for the top and
//            again for the bottom row;
//      16-bit: the box is 18 pixels wide, so that a row is 576 bytes = 64 mod 128: the top and
//            the bottom pair of corners (64 bytes each) fall into different halves of the banks
//            and ONE 128-bit load per lane fetches all four corners of the point without a
//            conflict -- lane = (row, side, channel half);
//    each lane accumulates its corner's (or corners') share for its channels in registers over
//    the nine taps; a few shuffles at the end add the corners up and every pair's channels are
//    stored once, 256 contiguous bytes per position;
//  * a point whose footprint leaves the box is gathered from global memory instead.
#include "tiled.cuh"

namespace dcnb200 {

namespace {

constexpr int kFwdTile = 8;      // positions per tile side
constexpr int kFwdGroups = 4;    // groups per task
constexpr int kFwdWarps = 8;
constexpr int kFwdThreads = kFwdWarps * 32;

template <typename T> struct FwdBox {
  static constexpr bool k16 = sizeof(T) == 2;
  static constexpr int BH = 16;
  static constexpr int BW = k16 ? 18 : 16;
  static constexpr int kPixel = 16 * (int)sizeof(T);          // bytes of a pixel's 16 channels
  static constexpr int kRow = BW * kPixel;                    // bytes of a box row
  static constexpr int kGroupBox = BH * kRow;                 // bytes of one group's box
  static constexpr int kVal = kFwdGroups * kGroupBox;
  // A patch of zeros behind the boxes: points that contribute nothing (outside the range test, or
  // pairs outside a ragged tile) read their "corners" here, so that 0 * value can never become NaN.
  static constexpr int kZero = (kRow + 2 * kPixel + 127) / 128 * 128;
  static constexpr int kOffZero = (kVal + 127) / 128 * 128;
  static constexpr int kRecOff = kFwdWarps * 32 * 4;          // int offset word per record
  static constexpr int kRecW = kFwdWarps * 32 * 16;           // four weights per record
  static constexpr int kOffRecOff = kOffZero + kZero;
  static constexpr int kOffRecW = kOffRecOff + kRecOff;
  static constexpr int kOffBar = kOffRecW + kRecW;
  static constexpr int kTotal = kOffBar + 16;
};

struct FwdTask {
  int b, g0, y0, x0, rows, cols, by0, bx0;
};

template <typename T>
__device__ __forceinline__ FwdTask fwd_task(int task, const DcnParams& p, int slices, int tiles_per_img) {
  using B = FwdBox<T>;
  FwdTask t;
  const int sl = task % slices;
  const int tile = task / slices;
  t.g0 = sl * kFwdGroups;
  t.b = tile / tiles_per_img;
  const int t_in = tile - t.b * tiles_per_img;
  const int tyi = t_in / p.tiles_x;
  t.y0 = tyi * kFwdTile;
  t.x0 = (t_in - tyi * p.tiles_x) * kFwdTile;
  t.rows = min(kFwdTile, p.Ho - t.y0);
  t.cols = min(kFwdTile, p.Wo - t.x0);
  // position (y, x) samples around pixel (y + 1 - ph, x + 1 - pw); the tile is centred in the box
  t.by0 = t.y0 + 1 - p.ph - ((B::BH - t.rows) >> 1);
  t.bx0 = t.x0 + 1 - p.pw - ((B::BW - t.cols) >> 1);
  return t;
}

template <typename T>
__global__ void __launch_bounds__(kFwdThreads, sizeof(T) == 4 ? 3 : 2)
dcnv4_fwd_tiled_kernel(const __grid_constant__ CUtensorMap vmap, const T* __restrict__ value,
                       const T* __restrict__ om, T* __restrict__ out, const DcnParams p, int n_tasks, int slices,
                       int* status) {
  using B = FwdBox<T>;
  constexpr bool k16 = B::k16;
  constexpr int NACC = k16 ? 8 : 4;  // channels a lane accumulates per pair
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_val = smem;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + B::kOffBar);

  const int lane = (int)threadIdx.x & 31, warp = (int)threadIdx.x >> 5;
  int* s_off = reinterpret_cast<int*>(smem + B::kOffRecOff) + warp * 32;
  float4* s_w = reinterpret_cast<float4*>(smem + B::kOffRecW) + warp * 32;
  const int quad = lane >> 3;  // which of the four points of a step this lane works on = its group in the slice
  // byte offset of this lane's first load relative to the point's top-left corner, the corner
  // weight(s) it uses, and where its group's box starts
  int lane_off, wsel;
  if constexpr (k16) {
    const int r = (lane >> 2) & 1, s = (lane >> 1) & 1, h = lane & 1;
    lane_off = r * B::kRow + s * B::kPixel + h * 16;
    wsel = r * 2 + s;                    // weights are stored {TL, TR, BL, BR}
  } else {
    const int s = (lane >> 2) & 1, cq = lane & 3;
    lane_off = s * B::kPixel + cq * 16;
    wsel = s;                            // this lane uses weights [s] (top) and [2 + s] (bottom)
  }
  const unsigned char* my_box = s_val + quad * B::kGroupBox + lane_off;

  static_assert(B::kGroupBox % 128 == 0 && B::kOffZero % 128 == 0, "record words keep their flag bits clear");
  if (threadIdx.x == 0) mbar_init(bar, 1);
  for (int i = (int)threadIdx.x; i < B::kZero / 4; i += kFwdThreads) reinterpret_cast<uint32_t*>(smem + B::kOffZero)[i] = 0u;
  __syncthreads();
  pdl_trigger();
  pdl_wait();  // value and offset_mask are the previous kernels' outputs

  const int tiles_per_img = p.tiles_x * p.tiles_y;
  const float Hf = (float)p.H, Wf = (float)p.W;
  const size_t img_elems = (size_t)p.H * p.W * p.C;
  const int row_elems = p.W * p.C;

  int task = (int)blockIdx.x;
  if (task < n_tasks && threadIdx.x == 0) {
    const FwdTask t0 = fwd_task<T>(task, p, slices, tiles_per_img);
    mbar_expect_tx(bar, (uint32_t)B::kVal);
    for (int g = 0; g < kFwdGroups; ++g)
      tma_load_4d(s_val + g * B::kGroupBox, &vmap, (t0.g0 + g) * 16, t0.bx0, t0.by0, t0.b, bar);
  }

  for (int it = 0; task < n_tasks; task += (int)gridDim.x, ++it) {
    const FwdTask t = fwd_task<T>(task, p, slices, tiles_per_img);
    // phase A role: lane l prepares pair l of this warp's tile row: position (row `warp`, column l / 4), group l % 4
    const int ga = t.g0 + (lane & 3);
    const int xa = t.x0 + (lane >> 2), ya = t.y0 + warp;
    const bool pair_ok = warp < t.rows && (lane >> 2) < t.cols;
    const T* om_row = om + (((size_t)t.b * p.Ho + (pair_ok ? ya : t.y0)) * p.Wo + (pair_ok ? xa : t.x0)) * p.Ppad + ga * 27;
    const float base_w = dcn_base(1 - p.pw + xa, 1, p.scale), base_h = dcn_base(1 - p.ph + ya, 1, p.scale);
    // global-memory view of this lane's channels for points that leave the box (roles of phase B)
    const T* img = value + (size_t)t.b * img_elems + (t.g0 + quad) * 16;

    float acc[kFwdTile][NACC];
#pragma unroll
    for (int j = 0; j < kFwdTile; ++j)
#pragma unroll
      for (int e = 0; e < NACC; ++e) acc[j][e] = 0.f;

    // tap 0's offsets and mask; the wait for the box comes after the loads are on their way
    float ox = 0.f, oy = 0.f, mk = 0.f;
    if (pair_ok) { ox = to_f32(om_row[0]); oy = to_f32(om_row[1]); mk = to_f32(om_row[18]); }
    if (!mbar_wait_bounded(bar, (uint32_t)(it & 1))) atomicExch(status, kStatusStageTimeout);

#pragma unroll 1
    for (int k = 0; k < 9; ++k) {
      float ox_n = 0.f, oy_n = 0.f, mk_n = 0.f;
      if (k < 8 && pair_ok) {
        ox_n = to_f32(om_row[2 * k + 2]); oy_n = to_f32(om_row[2 * k + 3]); mk_n = to_f32(om_row[19 + k]);
      }
      // ---- this lane's point of tap k
      {
        const int ti = (k * 11) >> 5, tj = k - 3 * ti;  // k = ti*3 + tj, ti over kernel_w
        const float w_im = dcn_coord(base_w, (float)ti, ox, p.scale);
        const float h_im = dcn_coord(base_h, (float)tj, oy, p.scale);
        int word = B::kOffZero - (lane & 3) * B::kGroupBox;  // the patch of zeros, seen from this pair's group box
        float4 wts = make_float4(0.f, 0.f, 0.f, 0.f);
        if (pair_ok && in_range(h_im, w_im, Hf, Wf)) {
          const float hf = floorf(h_im), wf = floorf(w_im);
          const int h0 = int_of_integral(hf), w0 = int_of_integral(wf);
          const float lh = h_im - hf, lw = w_im - wf, hh = 1.f - lh, hw = 1.f - lw;
          const float a = mk * hh, b = mk * lh;
          wts = make_float4(a * hw, a * lw, b * hw, b * lw);  // TL, TR, BL, BR
          const int rr = h0 - t.by0, cc = w0 - t.bx0;
          if (rr >= 0 && rr < B::BH - 1 && cc >= 0 && cc < B::BW - 1)
            word = rr * B::kRow + cc * B::kPixel;
          else
            word = (int)(((unsigned)(h0 + 1) << 19) | ((unsigned)(w0 + 1) << 6) | (unsigned)kRecOutside);
        }
        s_off[lane] = word;
        s_w[lane] = wts;
      }
      __syncwarp();
      // ---- eight steps of four points: step j = position j of the row, quarter-warp = group
      int anyout = 0;
#pragma unroll
      for (int j = 0; j < kFwdTile; ++j) anyout |= s_off[j * 4 + quad];
      const bool slow = __any_sync(0xffffffffu, (anyout & kRecOutside) != 0);
      if (!slow) {
#pragma unroll
        for (int j = 0; j < kFwdTile; ++j) {
          const int word = s_off[j * 4 + quad];
          if constexpr (k16) {
            const float wgt = reinterpret_cast<const float*>(&s_w[j * 4 + quad])[wsel];
            const uint4 raw = *reinterpret_cast<const uint4*>(my_box + word);
            const uint32_t r4[4] = {raw.x, raw.y, raw.z, raw.w};
            float v[8];
            widen(r4, v, (const T*)nullptr);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[j][e] = fmaf(wgt, v[e], acc[j][e]);
          } else {
            const float* wp = reinterpret_cast<const float*>(&s_w[j * 4 + quad]);
            const float wt = wp[wsel], wb = wp[2 + wsel];
            const float4 vt = *reinterpret_cast<const float4*>(my_box + word);
            const float4 vb = *reinterpret_cast<const float4*>(my_box + word + B::kRow);
            acc[j][0] = fmaf(wt, vt.x, fmaf(wb, vb.x, acc[j][0]));
            acc[j][1] = fmaf(wt, vt.y, fmaf(wb, vb.y, acc[j][1]));
            acc[j][2] = fmaf(wt, vt.z, fmaf(wb, vb.z, acc[j][2]));
            acc[j][3] = fmaf(wt, vt.w, fmaf(wb, vb.w, acc[j][3]));
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < kFwdTile; ++j) {
          const int word = s_off[j * 4 + quad];
          const float* wp = reinterpret_cast<const float*>(&s_w[j * 4 + quad]);
          if (!(word & kRecOutside)) {
            if constexpr (k16) {
              const uint4 raw = *reinterpret_cast<const uint4*>(my_box + word);
              const uint32_t r4[4] = {raw.x, raw.y, raw.z, raw.w};
              float v[8];
              widen(r4, v, (const T*)nullptr);
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[j][e] = fmaf(wp[wsel], v[e], acc[j][e]);
            } else {
              const float4 vt = *reinterpret_cast<const float4*>(my_box + word);
              const float4 vb = *reinterpret_cast<const float4*>(my_box + word + B::kRow);
              acc[j][0] = fmaf(wp[wsel], vt.x, fmaf(wp[2 + wsel], vb.x, acc[j][0]));
              acc[j][1] = fmaf(wp[wsel], vt.y, fmaf(wp[2 + wsel], vb.y, acc[j][1]));
              acc[j][2] = fmaf(wp[wsel], vt.z, fmaf(wp[2 + wsel], vb.z, acc[j][2]));
              acc[j][3] = fmaf(wp[wsel], vt.w, fmaf(wp[2 + wsel], vb.w, acc[j][3]));
            }
          } else {
            // the footprint leaves the box: same lane roles, corners fetched from global memory
            const int h0 = (int)((unsigned)word >> 19) - 1, w0 = ((word >> 6) & 8191) - 1;
            if constexpr (k16) {
              const int r = (lane >> 2) & 1, s = (lane >> 1) & 1, h = lane & 1;
              const int hy = h0 + r, wx = w0 + s;
              const bool ok = hy >= 0 && hy < p.H && wx >= 0 && wx < p.W;
              float v[8];
              gather_corner<T, 8>(img + ((hy * p.W + wx) * p.C + h * 8), ok, v);
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[j][e] = fmaf(wp[wsel], v[e], acc[j][e]);
            } else {
              const int s = (lane >> 2) & 1, cq = lane & 3;
              const int wx = w0 + s;
              const bool okc = wx >= 0 && wx < p.W;
              const int idx = (h0 * p.W + wx) * p.C + cq * 4;
              float vt[4], vb[4];
              gather_corner<T, 4>(img + idx, okc && h0 >= 0, vt);
              gather_corner<T, 4>(img + (idx + row_elems), okc && h0 + 1 < p.H, vb);
#pragma unroll
              for (int e = 0; e < 4; ++e) acc[j][e] = fmaf(wp[wsel], vt[e], fmaf(wp[2 + wsel], vb[e], acc[j][e]));
            }
          }
        }
      }
      __syncwarp();  // the record buffer is rewritten for the next tap
      ox = ox_n; oy = oy_n; mk = mk_n;
    }

    // ---- every reader of the box is done with it: request the next task's
    __syncthreads();
    const int next = task + (int)gridDim.x;
    if (next < n_tasks && threadIdx.x == 0) {
      const FwdTask tn = fwd_task<T>(next, p, slices, tiles_per_img);
      mbar_expect_tx(bar, (uint32_t)B::kVal);
      for (int g = 0; g < kFwdGroups; ++g)
        tma_load_4d(s_val + g * B::kGroupBox, &vmap, (tn.g0 + g) * 16, tn.bx0, tn.by0, tn.b, bar);
    }

    // ---- add the corners up across lanes and store: position j of row `warp`, group `quad`
    if (warp < t.rows) {
      T* orow = out + (((size_t)t.b * p.Ho + t.y0 + warp) * p.Wo + t.x0) * p.C + (t.g0 + quad) * 16;
#pragma unroll
      for (int j = 0; j < kFwdTile; ++j) {
        if constexpr (k16) {
          // lanes (r, s, h): fold r (xor 4) keeping half of the channels, then s (xor 2) keeping half again
          const bool up = (lane >> 2) & 1;   // r
          float k4[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float send = up ? acc[j][e] : acc[j][4 + e];
            const float keep = up ? acc[j][4 + e] : acc[j][e];
            k4[e] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
          }
          const bool right = (lane >> 1) & 1;  // s
          float k2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float send = right ? k4[e] : k4[2 + e];
            const float keep = right ? k4[2 + e] : k4[e];
            k2[e] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
          }
          // this lane now holds channels h*8 + r*4 + s*2 + {0, 1} of the pair
          if (j < t.cols) {
            const int ch = (lane & 1) * 8 + (up ? 4 : 0) + (right ? 2 : 0);
            uint32_t packed[1];
            narrow(k2, packed, (const T*)nullptr);
            *reinterpret_cast<uint32_t*>(orow + (size_t)j * p.C + ch) = packed[0];
          }
        } else {
          float sum[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) sum[e] = acc[j][e] + __shfl_xor_sync(0xffffffffu, acc[j][e], 4);
          if (j < t.cols && !((lane >> 2) & 1)) {
            uint32_t packed[4];
            narrow(sum, packed, (const T*)nullptr);
            stg_raw(orow + (size_t)j * p.C + (lane & 3) * 4, packed);
          }
        }
      }
    }
  }
}

template <typename T>
cudaError_t launch_fwd_tiled(int dtype, const T* value, const T* om, T* out, DcnParams p, int* status, cudaStream_t s) {
  using B = FwdBox<T>;
  CUtensorMap map;
  if (!make_value_map(&map, dtype, value, p.N, p.H, p.W, p.C, B::BH, B::BW)) return cudaErrorNotSupported;
  p.th = p.tw = kFwdTile;
  p.tiles_y = (p.Ho + kFwdTile - 1) / kFwdTile;
  p.tiles_x = (p.Wo + kFwdTile - 1) / kFwdTile;
  const int slices = p.G / kFwdGroups;
  const long long n_tasks = (long long)p.N * p.tiles_x * p.tiles_y * slices;
  if (n_tasks >= (1LL << 31)) return cudaErrorNotSupported;
  static bool attr_set[64] = {false};  // per device; written with the same value by any thread
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  dev &= 63;
  if (!attr_set[dev]) {
    e = cudaFuncSetAttribute(dcnv4_fwd_tiled_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, B::kTotal);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(dcnv4_fwd_tiled_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  int per_sm = (int)((227u * 1024u) / (unsigned)(B::kTotal + 1024));
  const int by_regs = sizeof(T) == 4 ? 3 : 2;
  if (per_sm > by_regs) per_sm = by_regs;
  const long long want = (long long)p.sm_count * per_sm;
  const int grid = (int)(n_tasks < want ? n_tasks : want);
  return launch_overlapped(dcnv4_fwd_tiled_kernel<T>, dim3((unsigned)grid), dim3(kFwdThreads), (size_t)B::kTotal, s, map,
                           value, om, out, p, (int)n_tasks, slices, status);
}

}  // namespace

// Whether the tiled forward covers this configuration.
bool dcnv4_fwd_tiled_applies(const DcnParams& p) {
  return p.kh == 3 && p.kw == 3 && p.sh == 1 && p.sw == 1 && p.dh == 1 && p.dw == 1 && !p.remove_center &&
         !p.softmax && p.D == 16 && p.G % kFwdGroups == 0 && p.H <= kTiledMaxSide && p.W <= kTiledMaxSide;
}

cudaError_t launch_dcnv4_fwd_tiled(int dtype, const void* value, const void* om, void* out, const DcnParams& p,
                                   int* status, cudaStream_t s) {
  switch (dtype) {
    case 0: return launch_fwd_tiled<float>(dtype, (const float*)value, (const float*)om, (float*)out, p, status, s);
    case 1: return launch_fwd_tiled<__half>(dtype, (const __half*)value, (const __half*)om, (__half*)out, p, status, s);
    default:
      return launch_fwd_tiled<__nv_bfloat16>(dtype, (const __nv_bfloat16*)value, (const __nv_bfloat16*)om,
                                             (__nv_bfloat16*)out, p, status, s);
  }
}

}  // namespace dcnb200
