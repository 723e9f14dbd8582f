// DCNv4 backward, spatially tiled: the value tile AND an fp32 image of grad_value for the tile
// live in shared memory, so a tile's ~36 contributions per pixel collapse into one vector
// reduction per pixel of (tile + halo) instead of going to L2 one by one.
//
// Replaces, for the configuration every FlashInternImage layer uses (3x3, stride 1,
// dilation 1, 16 channels per group, no softmax, centre kept), the same reference code as
// dcnv4_bwd.cu: backward_kernel_dcn_warp_primitive and its launcher
// (DCNv4_op/src/cuda/dcnv4_col2im_cuda.cuh:20-472, helper DCNv4_op/src/cuda/common.h:100-212).
// Every other configuration keeps the kernel of dcnv4_bwd.cu.
//
// STATUS: opt-in (DCNV4B200_TILED=1), not the default.  Measured on B200 at 64x56x56x64 fp32 this
// kernel takes 680-750 us (8x8, 6x6 and 4x4 query tiles alike) against 385 us for the kernel of
// dcnv4_bwd.cu, which sends every contribution to L2 as a vector reduction.  It removes ~8/9 of
// those reductions, as intended, but exclusive ownership of an accumulator box means one warp per
// box, hence 5-10 warps per SM, and with so few warps every section below is bound by the
// latency of its own dependent instructions rather than by shared-memory bandwidth.
//
// One warp per task (tile, group); see tiled.cuh for the lane geometry.  Per sampling point a
// quarter-warp issues, for the top and for the bottom row of the bilinear footprint, one
// 128-bit load of the value span, one 128-bit load and one 128-bit store of the accumulator
// span: plain read-modify-write, no atomics.  That is safe because
//  * the accumulator box belongs to this warp alone (one warp per CTA), and
//  * the four points a warp handles in one instruction come from four different quadrants of
//    the tile (same kernel tap, queries half a tile apart), and the lanes that prepare their
//    records check them pairwise: points whose 2x2 footprints share a pixel get different
//    colours (rounds), and rounds run one after the other.
// With one warp per task there are only 5-8 warps on an SM, so the latency of every dependent
// instruction shows.  The work is therefore laid out for instruction-level parallelism:
//  1. the records of ALL points of a task are prepared first (three passes of global loads in
//     flight at a time), while the TMA load of the value box is still under way;
//  2. a step -- the nine taps of four queries, 36 points -- is straight-line code: nine record
//     loads and eighteen value loads up front, then the chain of accumulator updates (the only
//     part that must stay in order), then dot products, shuffles and deposits for all nine taps;
//  3. the next task's value box is requested before this task's accumulator box is flushed.
// After the last point the box is added to the fp32 accumulation buffer in global memory with
// red.global.add.v4.f32 -- pixels outside the image (zero padding) and pixels nothing was added
// to are skipped -- and cleared for the next task.
//
// The offset/mask gradients of a point are reduced over the eight lanes with three shuffles
// (each lane first folds its four channels; the partial sums t = hh*d_top + lh*d_bot and
// u = d_bot - d_top are then exchanged so that half of the lanes finish t and half finish u),
// collected per query in a small shared-memory slab and written out 27 values at a time.
#include "tiled.cuh"

namespace dcnb200 {

namespace {

constexpr int kSlabStride = 28;   // floats per query in the gradient slab (27 used; 28 keeps the four
                                  // queries of a step in different banks)
// groups of four points per task of a TILE x TILE tile: (TILE/2)^2 steps x 9 taps
constexpr int max_groups(int tile) { return ((tile + 1) / 2) * ((tile + 1) / 2) * 9; }
constexpr int kPassesInFlight = 3;

// Two points collide when their 2x2 footprints share a pixel: rows and columns of the top-left
// corners both differ by at most one.  Keys hold (row + 1) << 14 | (column + 1).
__device__ __forceinline__ bool footprints_touch(int a, int b) {
  return abs((a >> 14) - (b >> 14)) <= 1 && abs((a & 16383) - (b & 16383)) <= 1;
}

template <typename T, int BH, int BW>
struct BwdTiledSmem {
  static constexpr int kMaxGroups = max_groups(BH - 8);
  static constexpr int kVal = BH * BW * 16 * (int)sizeof(T);
  static constexpr int kAcc = BH * BW * 16 * (int)sizeof(float);
  static constexpr int kRec = kMaxGroups * 4 * 16;
  static constexpr int kSlab = 4 * kSlabStride * (int)sizeof(float);
  static constexpr int kOffAcc = (kVal + 127) / 128 * 128;
  static constexpr int kOffRec = kOffAcc + kAcc;
  static constexpr int kOffSlab = kOffRec + kRec;
  static constexpr int kOffBar = kOffSlab + kSlab;
  static constexpr int kTotal = kOffBar + 16;
};

template <typename T>
__device__ __forceinline__ float4 ldg_chan4(const T* p, bool ok) {
  float v[4];
  gather_corner<T, 4>(p, ok, v);
  return make_float4(v[0], v[1], v[2], v[3]);
}

__device__ __forceinline__ void axpy4(float4& a, float w, const float4& x) {
  a.x = fmaf(w, x.x, a.x); a.y = fmaf(w, x.y, a.y); a.z = fmaf(w, x.z, a.z); a.w = fmaf(w, x.w, a.w);
}
__device__ __forceinline__ float dot4(const float4& a, const float4& b) {
  return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, a.w * b.w)));
}

// Geometry of one task.
struct TaskGeo {
  int g, b, y0, x0, rows, cols, by0, bx0;
};

template <int BH, int BW>
__device__ __forceinline__ TaskGeo task_geometry(int task, const DcnParams& p, int tiles_per_img) {
  TaskGeo t;
  t.g = task % p.G;
  const int tile = task / p.G;
  t.b = tile / tiles_per_img;
  const int t_in = tile - t.b * tiles_per_img;
  const int tyi = t_in / p.tiles_x;
  t.y0 = tyi * p.th;
  t.x0 = (t_in - tyi * p.tiles_x) * p.tw;
  t.rows = min(p.th, p.Ho - t.y0);
  t.cols = min(p.tw, p.Wo - t.x0);
  // box origin: query (y, x) samples around pixel (y + 1 - ph, x + 1 - pw); the tile is centred
  t.by0 = t.y0 + 1 - p.ph - ((BH - t.rows) >> 1);
  t.bx0 = t.x0 + 1 - p.pw - ((BW - t.cols) >> 1);
  return t;
}

template <typename T, int BH, int BW>
__global__ void __launch_bounds__(32)
dcnv4_bwd_tiled_kernel(const __grid_constant__ CUtensorMap vmap, const T* __restrict__ value,
                       const T* __restrict__ om, const T* __restrict__ gout, float* __restrict__ gvalue,
                       T* __restrict__ gom, const DcnParams p, int n_tasks, int* status) {
  using S = BwdTiledSmem<T, BH, BW>;
  constexpr int kRowBytes = BW * 64;  // one box row in the fp32 geometry
  extern __shared__ __align__(128) unsigned char smem[];
  T* s_val = reinterpret_cast<T*>(smem);
  float* s_acc = reinterpret_cast<float*>(smem + S::kOffAcc);
  int4* s_rec = reinterpret_cast<int4*>(smem + S::kOffRec);
  float* s_slab = reinterpret_cast<float*>(smem + S::kOffSlab);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + S::kOffBar);

  const int lane = (int)threadIdx.x;
  const int quad = lane >> 3, side = (lane >> 2) & 1, cq = lane & 3;  // roles while consuming records
  const int lane_off = side * 64 + cq * 16;
  // weight of this lane's corner column: lw on the right, 1 - lw on the left
  const float side_a = side ? 1.f : -1.f, side_b = side ? 0.f : 1.f;
  if (lane == 0) mbar_init(bar, 1);
  for (int i = lane; i < S::kAcc / 16; i += 32) sts_f4(s_acc, i * 16, make_float4(0.f, 0.f, 0.f, 0.f));
  __syncwarp();

  const int tiles_per_img = p.tiles_x * p.tiles_y;
  const int used = 27 * p.G;
  const float Hf = (float)p.H, Wf = (float)p.W;
  const size_t img_elems = (size_t)p.H * p.W * p.C;
  const int row_elems = p.W * p.C;

  int task = (int)blockIdx.x;
  if (task < n_tasks && lane == 0) {
    const TaskGeo t0 = task_geometry<BH, BW>(task, p, tiles_per_img);
    mbar_expect_tx(bar, (uint32_t)S::kVal);
    tma_load_4d(s_val, &vmap, t0.g * 16, t0.bx0, t0.by0, t0.b, bar);
  }

  for (int it = 0; task < n_tasks; task += (int)gridDim.x, ++it) {
    const TaskGeo tg = task_geometry<BH, BW>(task, p, tiles_per_img);
    const int g = tg.g, b = tg.b, y0 = tg.y0, x0 = tg.x0, rows = tg.rows, cols = tg.cols;
    const int by0 = tg.by0, bx0 = tg.bx0;
    // four quadrants of rows_a x cols_a queries; step i visits the i-th query of each quadrant
    const int rows_a = (rows + 1) >> 1, cols_a = (cols + 1) >> 1;
    const int inv_ca = (65536 + cols_a - 1) / cols_a;
    const int n_steps = rows_a * cols_a;
    const int n_grp = n_steps * 9;  // groups of four points (one per quadrant, same tap)
    const T* img = value + (size_t)b * img_elems + g * 16 + cq * 4;
    float* gimg = gvalue + (size_t)b * img_elems + g * 16 + cq * 4;
    const size_t q_img = (size_t)b * p.Ho * p.Wo;

    // ---- records of every point of the task: one per lane and pass, 8 groups x 4 quadrants a pass
    for (int grp0 = 0; grp0 < n_grp; grp0 += 8 * kPassesInFlight) {
      float ox[kPassesInFlight], oy[kPassesInFlight], mk[kPassesInFlight];
      int yy[kPassesInFlight], xx[kPassesInFlight], kk[kPassesInFlight];
      bool valid[kPassesInFlight];
      const int qa = lane & 3;
#pragma unroll
      for (int j = 0; j < kPassesInFlight; ++j) {
        const int grp = grp0 + 8 * j + (lane >> 2);
        const int i = grp / 9, k = grp - 9 * i;
        const int ri = (i * inv_ca) >> 16, ci = i - ri * cols_a;
        const int r = ri + (qa >> 1) * rows_a, c = ci + (qa & 1) * cols_a;
        valid[j] = grp < n_grp && r < rows && c < cols;
        yy[j] = y0 + r; xx[j] = x0 + c; kk[j] = k;
        ox[j] = oy[j] = mk[j] = 0.f;
        if (valid[j]) {
          const T* row = om + (q_img + (size_t)yy[j] * p.Wo + xx[j]) * p.Ppad + g * 27;
          ox[j] = to_f32(row[2 * k]);
          oy[j] = to_f32(row[2 * k + 1]);
          mk[j] = to_f32(row[18 + k]);
        }
      }
#pragma unroll
      for (int j = 0; j < kPassesInFlight; ++j) {
        if (grp0 + 8 * j >= n_grp) break;  // uniform
        int word = kRecDead;
        int key = -(lane + 1) * (4 << 14);  // a row of its own: touches nothing
        float lh = 0.f, lw = 0.f;
        if (valid[j]) {
          const int k = kk[j];
          const int ti = (k * 11) >> 5, tj = k - 3 * ti;  // k = ti*3 + tj, ti over kernel_w
          const float w_im = dcn_coord(dcn_base(1 - p.pw + xx[j], 1, p.scale), (float)ti, ox[j], p.scale);
          const float h_im = dcn_coord(dcn_base(1 - p.ph + yy[j], 1, p.scale), (float)tj, oy[j], p.scale);
          if (in_range(h_im, w_im, Hf, Wf)) {
            const float hf = floorf(h_im), wf = floorf(w_im);
            const int h0 = int_of_integral(hf), w0 = int_of_integral(wf);
            lh = h_im - hf; lw = w_im - wf;
            const int rr = h0 - by0, cc = w0 - bx0;
            if (rr >= 0 && rr < BH - 1 && cc >= 0 && cc < BW - 1) {
              word = (rr * BW + cc) * 64;
              key = ((h0 + 1) << 14) | (w0 + 1);
            } else {
              word = (int)(((unsigned)(h0 + 1) << 19) | ((unsigned)(w0 + 1) << 6) | (unsigned)kRecOutside);
            }
          }
        }
        // colour the group's four points: each takes the smallest round that no earlier point it
        // touches has taken
        const int base = lane & ~3;
        const int k0 = __shfl_sync(0xffffffffu, key, base), k1 = __shfl_sync(0xffffffffu, key, base + 1);
        const int k2 = __shfl_sync(0xffffffffu, key, base + 2), k3 = __shfl_sync(0xffffffffu, key, base + 3);
        const int r1 = footprints_touch(k0, k1) ? 1 : 0;
        const int m2 = (footprints_touch(k0, k2) ? 1 : 0) | (footprints_touch(k1, k2) ? (1 << r1) : 0);
        const int r2 = __ffs(~m2) - 1;
        const int m3 = (footprints_touch(k0, k3) ? 1 : 0) | (footprints_touch(k1, k3) ? (1 << r1) : 0) |
                       (footprints_touch(k2, k3) ? (1 << r2) : 0);
        const int r3 = __ffs(~m3) - 1;
        const int mine = qa == 0 ? 0 : (qa == 1 ? r1 : (qa == 2 ? r2 : r3));
        const int rounds = max(max(r1, r2), r3);
        word |= (mine << kRecRoundShift) | (rounds << kRecRoundsShift);
        s_rec[(grp0 + 8 * j) * 4 + lane] = make_int4(word, __float_as_int(lh), __float_as_int(lw), __float_as_int(mk[j]));
      }
    }

    if (!mbar_wait_bounded(bar, (uint32_t)(it & 1))) atomicExch(status, kStatusStageTimeout);
    __syncwarp();

    // this quarter-warp's query of step 0
    bool validq;
    size_t qidx;
    float4 gy;
    {
      const int r = (quad >> 1) * rows_a, c = (quad & 1) * cols_a;
      validq = r < rows && c < cols;
      qidx = q_img + (size_t)(y0 + (validq ? r : 0)) * p.Wo + (x0 + (validq ? c : 0));
      gy = ldg_chan4<T>(gout + qidx * p.C + g * 16 + cq * 4, validq);
    }

    for (int step = 0; step < n_steps; ++step) {
      // the next step's query: its grad_output channels are fetched now and used a step later
      bool validq_n = false;
      size_t qidx_n = 0;
      float4 gy_n = make_float4(0.f, 0.f, 0.f, 0.f);
      if (step + 1 < n_steps) {
        const int i = step + 1;
        const int ri = (i * inv_ca) >> 16, ci = i - ri * cols_a;
        const int r = ri + (quad >> 1) * rows_a, c = ci + (quad & 1) * cols_a;
        validq_n = r < rows && c < cols;
        qidx_n = q_img + (size_t)(y0 + (validq_n ? r : 0)) * p.Wo + (x0 + (validq_n ? c : 0));
        gy_n = ldg_chan4<T>(gout + qidx_n * p.C + g * 16 + cq * 4, validq_n);
      }

      const int4* recs = s_rec + step * 36 + quad;
      int4 rec[9];
#pragma unroll
      for (int k = 0; k < 9; ++k) rec[k] = recs[k * 4];
      int special = 0;
#pragma unroll
      for (int k = 0; k < 9; ++k) special |= rec[k].x;
      // outside the box, or a third colour: rare, taken through the general code below
      const bool slow = __any_sync(0xffffffffu, (special & (kRecOutside | (2 << kRecRoundShift))) != 0);
      float* slab = s_slab + quad * kSlabStride;

      if (!slow) {
        float4 vt[9], vb[9];
#pragma unroll
        for (int k = 0; k < 9; ++k) {
          const int off = (rec[k].x & 0xffc0) + lane_off;
          vt[k] = lds_val4(s_val, off);
          vb[k] = lds_val4(s_val, off + kRowBytes);
        }
        // accumulator updates, in order: colour 0 of tap 0, colour 1 of tap 0, colour 0 of tap 1, ...
#pragma unroll
        for (int k = 0; k < 9; ++k) {
          const int word = rec[k].x;
          const bool live = !(word & kRecDead);
          const int off = (word & 0xffc0) + lane_off;
          const float lh = __int_as_float(rec[k].y), lw = __int_as_float(rec[k].z), m = __int_as_float(rec[k].w);
          const float wside = fmaf(side_a, lw, side_b);
          const float wt = (m * (1.f - lh)) * wside, wb = (m * lh) * wside;
          if (live && !(word & (1 << kRecRoundShift))) {
            float4 at = lds_f4(s_acc, off), ab = lds_f4(s_acc, off + kRowBytes);
            axpy4(at, wt, gy);
            axpy4(ab, wb, gy);
            sts_f4(s_acc, off, at);
            sts_f4(s_acc, off + kRowBytes, ab);
          }
          __syncwarp();
          if (word & (3 << kRecRoundsShift)) {  // the group has a second colour (same answer in all lanes)
            if (live && (word & (1 << kRecRoundShift))) {
              float4 at = lds_f4(s_acc, off), ab = lds_f4(s_acc, off + kRowBytes);
              axpy4(at, wt, gy);
              axpy4(ab, wb, gy);
              sts_f4(s_acc, off, at);
              sts_f4(s_acc, off + kRowBytes, ab);
            }
            __syncwarp();
          }
        }
        // offset / mask gradients of the nine taps
#pragma unroll
        for (int k = 0; k < 9; ++k) {
          const bool live = !(rec[k].x & kRecDead);
          const float lh = __int_as_float(rec[k].y), lw = __int_as_float(rec[k].z), m = __int_as_float(rec[k].w);
          const float dt = dot4(gy, vt[k]), db = dot4(gy, vb[k]);
          const float t = fmaf(1.f - lh, dt, lh * db), u = db - dt;
          // fold the four channel lanes of each side: even lanes finish t, odd lanes finish u
          const float send = (cq & 1) ? t : u;
          float keep = ((cq & 1) ? u : t) + __shfl_xor_sync(0xffffffffu, send, 1);
          keep += __shfl_xor_sync(0xffffffffu, keep, 2);
          const float other = __shfl_xor_sync(0xffffffffu, keep, 4);
          // lane 0: keep = T_left, other = T_right; lane 1: keep = U_left, other = U_right
          const float sm = p.scale * m;
          const float diff = sm * (other - keep);                 // lane 0: d/dx
          const float mix = fmaf(lw, other, (1.f - lw) * keep);   // lane 0: d/dmask; lane 1: d/dy before sm
          if (side == 0 && cq < 2) slab[2 * k + cq] = live ? (cq == 0 ? diff : sm * mix) : 0.f;
          if (side == 0 && cq == 0) slab[18 + k] = live ? mix : 0.f;
        }
      } else {
        for (int k = 0; k < 9; ++k) {
          const int4 rk = recs[k * 4];
          const int word = rk.x;
          const bool live = !(word & kRecDead);
          const int my_round = (word >> kRecRoundShift) & 3;
          const int rounds = (word >> kRecRoundsShift) & 3;  // same in the four records of a group
          const float lh = __int_as_float(rk.y), lw = __int_as_float(rk.z), m = __int_as_float(rk.w);
          const float hh = 1.f - lh, hw = 1.f - lw;
          const float wside = fmaf(side_a, lw, side_b);
          const float wt = (m * hh) * wside, wb = (m * lh) * wside;
          float t = 0.f, u = 0.f;
          for (int rd = 0; rd <= rounds; ++rd) {
            if (live && my_round == rd) {
              float4 vt, vb;
              if (!(word & kRecOutside)) {
                const int off = (word & 0xffc0) + lane_off;
                vt = lds_val4(s_val, off);
                vb = lds_val4(s_val, off + kRowBytes);
                float4 at = lds_f4(s_acc, off), ab = lds_f4(s_acc, off + kRowBytes);
                axpy4(at, wt, gy);
                axpy4(ab, wb, gy);
                sts_f4(s_acc, off, at);
                sts_f4(s_acc, off + kRowBytes, ab);
              } else {
                const int h0 = (int)((unsigned)word >> 19) - 1, w0 = ((word >> 6) & 8191) - 1;
                const int col = w0 + side;
                const bool okc = col >= 0 && col < p.W;
                const bool okt = okc && h0 >= 0, okb = okc && h0 + 1 < p.H;
                const int idx = (h0 * p.W + col) * p.C;
                vt = ldg_chan4<T>(img + idx, okt);
                vb = ldg_chan4<T>(img + (idx + row_elems), okb);
                if (okt) red_add_v4(gimg + idx, wt * gy.x, wt * gy.y, wt * gy.z, wt * gy.w);
                if (okb) red_add_v4(gimg + (idx + row_elems), wb * gy.x, wb * gy.y, wb * gy.z, wb * gy.w);
              }
              const float dt = dot4(gy, vt), db = dot4(gy, vb);
              t = fmaf(hh, dt, lh * db);
              u = db - dt;
            }
            __syncwarp();
          }
          const float send = (cq & 1) ? t : u;
          float keep = ((cq & 1) ? u : t) + __shfl_xor_sync(0xffffffffu, send, 1);
          keep += __shfl_xor_sync(0xffffffffu, keep, 2);
          const float other = __shfl_xor_sync(0xffffffffu, keep, 4);
          const float sm = p.scale * m;
          const float diff = sm * (other - keep);
          const float mix = fmaf(lw, other, hw * keep);
          if (side == 0 && cq < 2) slab[2 * k + cq] = live ? (cq == 0 ? diff : sm * mix) : 0.f;
          if (side == 0 && cq == 0) slab[18 + k] = live ? mix : 0.f;
        }
      }

      // the step's four queries are complete: 27 gradient values each
      __syncwarp();
      if (validq) {
        T* grow = gom + qidx * p.Ppad;
        const int l8 = lane & 7;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (l8 + 8 * e < 27) grow[g * 27 + l8 + 8 * e] = from_f32<T>(slab[l8 + 8 * e]);
        if (g == p.G - 1)  // pad columns of the row are zeros
          for (int e = used + l8; e < p.Ppad; e += 8) grow[e] = from_f32<T>(0.f);
      }
      __syncwarp();
      validq = validq_n; qidx = qidx_n; gy = gy_n;
    }

    // ---- the value box is free: request the next task's while this task's accumulator box drains
    const int next = task + (int)gridDim.x;
    if (next < n_tasks && lane == 0) {
      const TaskGeo tn = task_geometry<BH, BW>(next, p, tiles_per_img);
      mbar_expect_tx(bar, (uint32_t)S::kVal);
      tma_load_4d(s_val, &vmap, tn.g * 16, tn.bx0, tn.by0, tn.b, bar);
    }

    // ---- add the box to the global accumulation buffer and clear it
#pragma unroll 4
    for (int pix = lane >> 2; pix < BH * BW; pix += 8) {
      const int rr = pix / BW, cc = pix - rr * BW;
      const int y = by0 + rr, x = bx0 + cc;
      const int off = pix * 64 + cq * 16;
      const float4 a = lds_f4(s_acc, off);
      const bool any = a.x != 0.f || a.y != 0.f || a.z != 0.f || a.w != 0.f;
      if (any) {
        if (y >= 0 && y < p.H && x >= 0 && x < p.W)
          red_add_v4(gimg + ((size_t)y * p.W + x) * p.C, a.x, a.y, a.z, a.w);
        sts_f4(s_acc, off, make_float4(0.f, 0.f, 0.f, 0.f));
      }
    }
    __syncwarp();
  }
}

template <typename T, int BH, int BW>
cudaError_t launch_tiled(int dtype, const T* value, const T* om, const T* gout, float* gvalue, T* gom, DcnParams p,
                         int* status, cudaStream_t s) {
  using S = BwdTiledSmem<T, BH, BW>;
  CUtensorMap map;
  if (!make_value_map(&map, dtype, value, p.N, p.H, p.W, p.C, BH, BW)) return cudaErrorNotSupported;
  p.th = tiled_tile_extent(p.Ho, BH - 8);
  p.tw = tiled_tile_extent(p.Wo, BW - 8);
  p.tiles_y = (p.Ho + p.th - 1) / p.th;
  p.tiles_x = (p.Wo + p.tw - 1) / p.tw;
  const long long n_tasks = (long long)p.N * p.tiles_x * p.tiles_y * p.G;
  if (n_tasks >= (1LL << 31)) return cudaErrorNotSupported;
  static_assert(S::kTotal <= 48 * 1024, "the box must fit the default dynamic shared-memory limit");
  int per_sm = (int)((227u * 1024u) / (unsigned)(S::kTotal + 1024));
  if (per_sm > 32) per_sm = 32;
  // One-warp CTAs with 34-43 KB each: without this hint the driver may size the shared-memory
  // carve-out for fewer resident CTAs than fit.
  static bool carveout_set[64] = {false};  // per device; written with the same value by any thread
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  dev &= 63;
  if (!carveout_set[dev]) {
    e = cudaFuncSetAttribute(dcnv4_bwd_tiled_kernel<T, BH, BW>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    carveout_set[dev] = true;
  }
  const long long want = (long long)p.sm_count * per_sm;
  const int grid = (int)(n_tasks < want ? n_tasks : want);
  dcnv4_bwd_tiled_kernel<T, BH, BW><<<grid, 32, S::kTotal, s>>>(map, value, om, gout, gvalue, gom, p, (int)n_tasks, status);
  return cudaGetLastError();
}

}  // namespace

bool make_value_map(CUtensorMap* m, int dtype, const void* base, int N, int H, int W, int C, int box_h, int box_w) {
  using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiledFn enc = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  if (!enc) return false;
  const cuuint64_t es = dtype == 0 ? 4 : 2;
  const cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  const cuuint64_t strides[3] = {(cuuint64_t)C * es, (cuuint64_t)W * C * es, (cuuint64_t)H * W * C * es};
  const cuuint32_t box[4] = {16u, (cuuint32_t)box_w, (cuuint32_t)box_h, 1u};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                            : (dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  return enc(m, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Whether the tiled kernel covers this configuration.
bool dcnv4_bwd_tiled_applies(const DcnParams& p) {
  return p.kh == 3 && p.kw == 3 && p.sh == 1 && p.sw == 1 && p.dh == 1 && p.dw == 1 && !p.remove_center &&
         !p.softmax && p.D == 16 && p.H <= kTiledMaxSide && p.W <= kTiledMaxSide;
}

cudaError_t launch_dcnv4_bwd_tiled(int dtype, const void* value, const void* om, const void* gout,
                                   float* gvalue_f32, void* gom, const DcnParams& p, int* status, cudaStream_t s) {
  switch (dtype) {
    case 0:
      return launch_tiled<float, 16, 16>(dtype, (const float*)value, (const float*)om, (const float*)gout, gvalue_f32,
                                         (float*)gom, p, status, s);
    case 1:
      return launch_tiled<__half, 16, 16>(dtype, (const __half*)value, (const __half*)om, (const __half*)gout,
                                          gvalue_f32, (__half*)gom, p, status, s);
    default:
      return launch_tiled<__nv_bfloat16, 16, 16>(dtype, (const __nv_bfloat16*)value, (const __nv_bfloat16*)om,
                                                 (const __nv_bfloat16*)gout, gvalue_f32, (__nv_bfloat16*)gom, p,
                                                 status, s);
  }
}

}  // namespace dcnb200
