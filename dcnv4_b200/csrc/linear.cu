// Linear layer with a fused epilogue on the 5th-generation tensor cores (tcgen05, sm_100a):
//
//     y[m, :] = epilogue( x[m, :] . W^T + bias )           x (M,K), W (N,K), y (M,N), 16-bit
//
// FlashInternImage wraps every DCNv4 operator in 1x1 projections and an MLP whose GELU and
// residual additions the reference runs as separate element-wise kernels
// (classification/models/flash_intern_image.py:308-341 MLPLayer, :414-432 residual adds).  At
// inference those kernels move more bytes than the matrix products they follow.  Here the
// activation / residual is applied to the accumulator on its way out of tensor memory, so the
// intermediate never goes to HBM.
//
// One persistent CTA per SM, eighteen warps with fixed roles:
//   warp 0     producer : TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) loads of the x tile
//                         (128 x 64) and W tile (BN x 64) into a shared-memory ring;
//   warp 1     MMA      : one elected lane issues tcgen05.mma (M=128, N=BN, K=16, fp32
//                         accumulate) from shared-memory descriptors into one of two
//                         accumulators in tensor memory; tcgen05.commit frees ring slots and
//                         publishes finished accumulators;
//   warps 2-17 epilogue : tcgen05.ld of the accumulator (warp%4 selects the 32-lane quadrant a
//                         warp may read, the other two bits a group of columns), bias, rounding
//                         to the storage type, GELU by table, residual; the result goes to a
//                         swizzled staging tile and leaves through a TMA store, which writes
//                         whole lines and clips the ragged edge of the matrix.  The residual
//                         tile arrives by TMA load into the same staging tile.  Optionally the
//                         LayerNorm of the finished row leaves as a second output (ACT == 2),
//                         or the columns beyond `n_split` go to a second tensor (two stacked
//                         layers in one product).
//                         64-column tiles need only eight of these warps; the other eight then
//                         form a second set working on the other accumulator.
// The double-buffered accumulator lets the epilogue of tile i overlap the products of tile
// i+1.  Every mbarrier wait is bounded; a wait that runs out records kStatusStageTimeout in
// the device status word, the roles leave their loops and the CTA frees its tensor memory.
//
// The epilogue, not the tensor pipe, bounds this kernel at the model's shapes (K = 64..512,
// so a 128 x 256 tile needs only 4-32 MMA instructions but 32768 activations); that is why it
// gets sixteen warps, why per-element work is kept to a table lookup for GELU, and why stores
// are left to the TMA unit instead of per-lane 16-byte writes to 32 different rows.
//
// Rounding mirrors the unfused module sequence: the product plus bias is rounded to the
// storage type first (what nn.Linear would have written), the activation or residual is then
// evaluated in fp32 on that rounded value and rounded once more.
//
// Building with -DDCNB200_LINEAR_PROFILE adds clock64() timers around the phases of each role
// (CTA 0 only) and an extra entry point, dcnv4b200_linear_profile, that returns them; it is a tuning
// aid, off by default, never part of a shipped build and deliberately not declared in
// include/dcnv4_b200.h: the header describes exactly what the default build exports.
#include <mutex>

#include "gelu_table.cuh"
#include "tc.cuh"

namespace dcnb200 {

namespace {

using namespace tc;

constexpr int kBM = 128;        // rows of x per tile == tensor-memory lanes
constexpr int kBK = 64;         // 64 16-bit elements == 128 bytes == one swizzle span
#ifndef DCNB200_LINEAR_EPI_WARPS
#define DCNB200_LINEAR_EPI_WARPS 16
#endif
constexpr int kEpiWarps = DCNB200_LINEAR_EPI_WARPS;  // 4 quadrants x column groups
constexpr int kGemmThreads = 32 * (2 + kEpiWarps);
constexpr int kUmmaK = 16;          // K of one tcgen05.mma for 16-bit operands
constexpr int kStagingTile = 4096;  // epilogue staging tile of one warp: 32 rows x (at most) 128 bytes
constexpr int kBarrierBytes = 512;

template <typename T, int ACT>
constexpr int lut_bytes() { return ACT == 1 ? gelu_lut_bytes<T>() : 0; }
// fp32 bias, gamma and beta of each epilogue warp's current 64 columns, then two arrays of
// per-row partial sums (one float per epilogue thread) for the LayerNorm epilogue
template <int ACT>
constexpr int bias_bytes() { return ACT == 2 ? kEpiWarps * 64 * 4 * 3 + 2 * kEpiWarps * 32 * 4 : kEpiWarps * 64 * 4; }

// Shared-memory ring depth: as many (x tile + W tile) slots as fit beside staging and table.
template <typename T, int BN, int ACT>
constexpr int stages() {
  constexpr int slot = kBM * kBK * 2 + BN * kBK * 2;
  constexpr int room = 227 * 1024 - 1024 - kBarrierBytes - bias_bytes<ACT>() - kEpiWarps * kStagingTile - lut_bytes<T, ACT>();
  return room / slot > 8 ? 8 : room / slot;
}
// Column groups the epilogue warps split a tile into (each at least 32 columns wide).
template <int BN>
constexpr int col_groups() { return kEpiWarps / 4 < BN / 32 ? kEpiWarps / 4 : BN / 32; }

struct LinearParams {
  long long M;
  int N, K;
  int m_tiles, n_tiles, k_blocks;
  const void* bias;      // (N) or null
  const void* residual;  // (M,N) or null
  const void* gamma;     // LayerNorm epilogue (ACT == 2): weight, bias (N), eps
  const void* beta;
  float eps;
  int n_split;           // > 0 (ACT == 0 only): columns [n_split, N) go to a second tensor (map_z)
  void* y;
  int* status;
};

template <typename T, int BN, int ACT>
constexpr size_t ring_bytes() { return (size_t)stages<T, BN, ACT>() * (kBM * kBK * 2 + BN * kBK * 2); }
template <typename T, int BN, int ACT>
constexpr size_t smem_bytes() {
  return ring_bytes<T, BN, ACT>() + kEpiWarps * kStagingTile + lut_bytes<T, ACT>() + bias_bytes<ACT>() + 1024 /*alignment slack*/ +
         kBarrierBytes;
}

// Columns of one epilogue staging unit: a warp's share of the tile, at most 64 (128 bytes).
template <int BN>
constexpr int unit_cols() { return BN / col_groups<BN>() < 64 ? BN / col_groups<BN>() : 64; }

#ifdef DCNB200_LINEAR_PROFILE
__device__ long long g_lin_prof[16];
#define PROF_T0() long long _t0 = clock64()
#define PROF_ADD(slot) do { long long _t1 = clock64(); if (blockIdx.x == 0) prof_acc[slot] += _t1 - _t0; _t0 = _t1; } while (0)
#else
#define PROF_T0() do {} while (0)
#define PROF_ADD(slot) do {} while (0)
#endif

// ---- kernel ------------------------------------------------------------------------------

template <typename T, int BN, int ACT>
__global__ void __launch_bounds__(kGemmThreads, 1)
linear_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
              const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_r,
              const __grid_constant__ CUtensorMap map_z, const LinearParams p) {
  extern __shared__ unsigned char smem_raw[];
  // 128-byte swizzled tiles must start on a 1024-byte boundary.
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr uint32_t kBytesA = kBM * kBK * 2, kBytesB = BN * kBK * 2;
  unsigned char* ring_a = smem;
  constexpr int kStages = stages<T, BN, ACT>();
  constexpr int kCG = col_groups<BN>();
  unsigned char* ring_b = smem + kStages * kBytesA;
  unsigned char* staging = smem + ring_bytes<T, BN, ACT>();
  uint16_t* lut = reinterpret_cast<uint16_t*>(staging + kEpiWarps * kStagingTile);
  float* bias_f32 = reinterpret_cast<float*>(staging + kEpiWarps * kStagingTile + lut_bytes<T, ACT>());
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kEpiWarps * kStagingTile + lut_bytes<T, ACT>() + bias_bytes<ACT>());
  uint64_t* full = bars;                  // [kStages] TMA landed
  uint64_t* empty = bars + kStages;       // [kStages] MMA finished reading
  uint64_t* acc_full = bars + 2 * kStages;      // [2] accumulator complete
  uint64_t* acc_empty = bars + 2 * kStages + 2; // [2] accumulator drained by the epilogue
  uint64_t* res_bars = bars + 2 * kStages + 4;  // [kEpiWarps] residual tile landed
  uint64_t* quad_bars = res_bars + kEpiWarps;    // [2 sets][4] LayerNorm epilogue: row partial sums published
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(quad_bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;  // power of two: BN in {32,64,128,256}

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4 * kCG); }
    for (int w = 0; w < kEpiWarps; ++w) mbar_init(&res_bars[w], 1);
    for (int q = 0; q < 8; ++q) mbar_init(&quad_bars[q], (uint32_t)((p.N + BN / kCG - 1) / (BN / kCG)));
    *abort_flag = 0;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();

  const long long n_tiles_total = (long long)p.m_tiles * p.n_tiles;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      pdl_wait();  // x may be the previous kernel's output
#ifdef DCNB200_LINEAR_PROFILE
      long long prof_acc[16] = {0};
#endif
      PROF_T0();
      for (long long t = blockIdx.x; t < n_tiles_total && !*abort_flag; t += gridDim.x) {
        const int mt = (int)(t / p.n_tiles), nt = (int)(t % p.n_tiles);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          PROF_ADD(0);
          if (!mbar_wait_bounded(&empty[stage], phase ^ 1)) { atomicExch(p.status, kStatusStageTimeout); *abort_flag = 1; break; }
          PROF_ADD(1);
          mbar_expect_tx(&full[stage], kBytesA + kBytesB);
          tma_load_2d(ring_a + stage * kBytesA, &map_x, kb * kBK, mt * kBM, &full[stage]);
          tma_load_2d(ring_b + stage * kBytesB, &map_w, kb * kBK, nt * BN, &full[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
#ifdef DCNB200_LINEAR_PROFILE
      if (blockIdx.x == 0) { g_lin_prof[0] = prof_acc[0]; g_lin_prof[1] = prof_acc[1]; }
#endif
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc<T>(BN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
#ifdef DCNB200_LINEAR_PROFILE
      long long prof_acc[16] = {0};
#endif
      PROF_T0();
      for (long long t = blockIdx.x; t < n_tiles_total && !*abort_flag; t += gridDim.x) {
        PROF_ADD(2);
        if (!mbar_wait_bounded(&acc_empty[acc], acc_phase ^ 1)) { atomicExch(p.status, kStatusStageTimeout); *abort_flag = 1; break; }
        PROF_ADD(3);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          PROF_ADD(2);
          if (!mbar_wait_bounded(&full[stage], phase)) { atomicExch(p.status, kStatusStageTimeout); *abort_flag = 1; break; }
          PROF_ADD(4);
          tc_fence_after();
          const uint64_t da = smem_desc_sw128(ring_a + stage * kBytesA);
          const uint64_t db = smem_desc_sw128(ring_b + stage * kBytesB);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)  // 32 bytes further along K inside the swizzle span
            tc_mma_f16(d_tmem, da + (uint64_t)(k * kUmmaK * 2 / 16), db + (uint64_t)(k * kUmmaK * 2 / 16), idesc,
                       (kb | k) != 0);
          tc_commit(&empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        tc_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
#ifdef DCNB200_LINEAR_PROFILE
      if (blockIdx.x == 0) { g_lin_prof[2] = prof_acc[2]; g_lin_prof[3] = prof_acc[3]; g_lin_prof[4] = prof_acc[4]; }
#endif
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    // Each lane owns one accumulator row (that is how tensor memory is read).  It applies bias,
    // rounding, activation and residual and parks 16-byte pieces in a staging tile laid out with
    // the TMA swizzle; one lane then hands the tile to a TMA store, which writes whole lines
    // and clips rows and columns beyond the matrix.  The residual tile arrives the same way
    // (TMA load into the staging tile, consumed in place).  Two staging tiles per warp let the
    // store of one unit overlap the arithmetic of the next.
    const int quad = warp & 3;              // tensor-memory lanes [32*quad, 32*quad+32)
    // A tile occupies 4 * kCG warps.  When that is only half of the epilogue warps (64-column
    // tiles) the other half forms a second set that takes every other tile -- and with it the
    // other accumulator -- so two epilogues are in flight and their latencies overlap.
    constexpr int kSets = kEpiWarps / (4 * kCG);
    const int set = ((warp - 2) >> 2) / kCG;
    const int group = ((warp - 2) >> 2) % kCG;  // which column group of the tile
    constexpr int kColsPerWarp = BN / kCG;
    constexpr int UW = unit_cols<BN>();     // columns per staging unit (32 or 64)
    constexpr int RB = UW * 2;        // bytes per staged row (64 or 128) == swizzle span
    constexpr int CPR = RB / 16;      // 16-byte pieces per row
    constexpr int RPW = 128 / RB;     // rows per 128-byte bank window
    unsigned char* buf = staging + (warp - 2) * kStagingTile;
    uint64_t* res_bar = &res_bars[warp - 2];
    constexpr int kParamFloats = ACT == 2 ? 192 : 64;  // [0,64) bias; LayerNorm: [64,128) gamma, [128,192) beta
    float* my_bias = bias_f32 + (warp - 2) * kParamFloats;
    float* stats = bias_f32 + kEpiWarps * kParamFloats;  // LayerNorm: [2][kEpiWarps * 32] per-row partial sums
    const T* bias = static_cast<const T*>(p.bias);
    const bool has_res = p.residual != nullptr;
    uint32_t unit = 0, ln_phase = 0;
    uint64_t* quad_bar = &quad_bars[set * 4 + quad];
    const int stat_slot = ((set * 4 + quad) * kCG) * 32 + lane;  // + group * 32
    if (ACT == 1) {
      // Fill the GELU table (epilogue warps only; the pipeline fills meanwhile).
      gelu_lut_fill<T>(lut, threadIdx.x - 64, 32 * kEpiWarps);
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
    }
    pdl_wait();  // residual may be the previous kernel's output; y may be read by it
#ifdef DCNB200_LINEAR_PROFILE
    long long prof_acc[16] = {0};
#endif
    PROF_T0();
    long long t = blockIdx.x;
    for (uint32_t it = 0; t < n_tiles_total && !*abort_flag; t += gridDim.x, ++it) {
      if (kSets > 1 && (int)(it % kSets) != set) continue;
      const int acc = (int)(it & 1);
      const uint32_t acc_phase = (it >> 1) & 1;
      const int mt = (int)(t / p.n_tiles), nt = (int)(t % p.n_tiles);
      PROF_ADD(5);
      if (!mbar_wait_bounded(&acc_full[acc], acc_phase)) {
        if (lane == 0) { atomicExch(p.status, kStatusStageTimeout); *abort_flag = 1; }
        break;
      }
      tc_fence_after();
      PROF_ADD(6);
      const int row0 = mt * kBM + quad * 32;
      // The residual tile is needed the moment the accumulator is read; fetching it from DRAM
      // only then would expose the full latency once per tile, so the next tile's residual is
      // pulled into L2 now, a whole tile ahead.
      if (has_res && lane == 0 && t + (long long)kSets * gridDim.x < n_tiles_total) {
        const long long tn = t + (long long)kSets * gridDim.x;
        const int mt_n = (int)(tn / p.n_tiles), nt_n = (int)(tn % p.n_tiles);
        for (int c = 0; c < kColsPerWarp; c += UW) {
          const int col_n = nt_n * BN + group * kColsPerWarp + c;
          if (col_n < p.N) tma_prefetch_2d(&map_r, col_n, mt_n * kBM + quad * 32);
        }
      }
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + group * kColsPerWarp);
#pragma unroll 1
      for (int c = 0; c < kColsPerWarp; c += UW, ++unit) {
        const int col0 = nt * BN + group * kColsPerWarp + c;
        if (col0 >= p.N) break;  // warp-uniform
        // The previous store read this tile; it must be done before we overwrite it.
        if (lane == 0) {
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          if (has_res) {
            mbar_expect_tx(res_bar, 32 * RB);
            tma_load_2d(buf, &map_r, col0, row0, res_bar);
          }
        }
        // Accumulator columns are fetched 32 at a time (32 registers); the first fetch is in
        // flight while the warp stages this unit's bias as fp32 (two columns per lane, zero
        // where there is none) so that the per-row loop reads it with 16-byte shared loads.
        uint32_t v[32];
        uint32_t yreg[ACT == 2 ? UW / 2 : 1];  // this lane's row of the result, kept for the LayerNorm pass
        tmem_ld_32x32(taddr0 + (uint32_t)c, v);
#pragma unroll
        for (int q = lane * 2; q < UW; q += 64) {
          const int col = col0 + q;
          float2 b = make_float2(0.f, 0.f);
          if (bias != nullptr && col < p.N) b = unpack2<T>(__ldg(reinterpret_cast<const uint32_t*>(bias + col)));
          *reinterpret_cast<float2*>(my_bias + q) = b;
          if (ACT == 2) {
            const T* gamma = static_cast<const T*>(p.gamma);
            const T* beta = static_cast<const T*>(p.beta);
            *reinterpret_cast<float2*>(my_bias + 64 + q) = unpack2<T>(__ldg(reinterpret_cast<const uint32_t*>(gamma + col)));
            *reinterpret_cast<float2*>(my_bias + 128 + q) = unpack2<T>(__ldg(reinterpret_cast<const uint32_t*>(beta + col)));
          }
        }
        __syncwarp();
        if (has_res && !mbar_wait_bounded(res_bar, unit & 1)) {
          if (lane == 0) { atomicExch(p.status, kStatusStageTimeout); *abort_flag = 1; }
        }
#pragma unroll
        for (int cc = 0; cc < UW; cc += 32) {
          if (cc > 0) tmem_ld_32x32(taddr0 + (uint32_t)(c + cc), v);
          tmem_ld_wait();
          PROF_ADD(7);
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            const float4 bA = *reinterpret_cast<const float4*>(my_bias + cc + j);
            const float4 bB = *reinterpret_cast<const float4*>(my_bias + cc + j + 4);
            const float b8[8] = {bA.x, bA.y, bA.z, bA.w, bB.x, bB.y, bB.z, bB.w};
            uint4* slot = reinterpret_cast<uint4*>(buf + lane * RB + ((((cc + j) >> 3) ^ ((lane / RPW) % CPR)) << 4));
            uint32_t r4[4] = {0u, 0u, 0u, 0u};
            if (has_res) { const uint4 r = *slot; r4[0] = r.x; r4[1] = r.y; r4[2] = r.z; r4[3] = r.w; }
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 8; e += 2)  // rounded to storage, as nn.Linear would write it
              o[e >> 1] = pack2<T>(__uint_as_float(v[j + e]) + b8[e], __uint_as_float(v[j + e + 1]) + b8[e + 1]);
            if (ACT == 1) gelu_lut8<T>(o, lut);
            if (has_res) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float2 h = unpack2<T>(o[q]);
                const float2 r = unpack2<T>(r4[q]);
                o[q] = pack2<T>(h.x + r.x, h.y + r.y);
              }
            }
            *slot = make_uint4(o[0], o[1], o[2], o[3]);
            if (ACT == 2) {
#pragma unroll
              for (int q = 0; q < 4; ++q) yreg[((cc + j) >> 1) + q] = o[q];
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        PROF_ADD(8);
        if (lane == 0) {
          if (ACT == 0 && p.n_split > 0 && col0 >= p.n_split) tma_store_2d(&map_z, buf, col0 - p.n_split, row0);
          else tma_store_2d(&map_y, buf, col0, row0);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        PROF_ADD(9);
        if (ACT == 2) {
          // LayerNorm of the row just produced (second output z).  A row's columns are spread
          // over the column-group warps of this quadrant; they exchange per-row partial sums
          // through shared memory and meet at an mbarrier (one per quadrant, one arrival per
          // warp that owns columns; bounded waits like everywhere else).  Each warp reduces its own
          // columns to (mean, sum of squared deviations) and the pairs are combined exactly
          // (Chan et al.), so one exchange per tile suffices and nothing cancels.
          const int n_groups = (p.N + kColsPerWarp - 1) / kColsPerWarp;  // groups that own columns
          // this warp's share of the row: mean and sum of squared deviations of its UW columns
          float s1 = 0.f;
#pragma unroll
          for (int q = 0; q < UW / 2; ++q) { const float2 f = unpack2<T>(yreg[q]); s1 += f.x + f.y; }
          const float m_loc = s1 * (1.f / (float)UW);
          float s2 = 0.f;
#pragma unroll
          for (int q = 0; q < UW / 2; ++q) {
            const float2 f = unpack2<T>(yreg[q]);
            s2 = fmaf(f.x - m_loc, f.x - m_loc, s2);
            s2 = fmaf(f.y - m_loc, f.y - m_loc, s2);
          }
          stats[stat_slot + group * 32] = m_loc;
          stats[kEpiWarps * 32 + stat_slot + group * 32] = s2;
          __syncwarp();
          if (lane == 0) mbar_arrive(quad_bar);
          if (!mbar_wait_bounded(quad_bar, ln_phase) && lane == 0) { atomicExch(p.status, kStatusStageTimeout); *abort_flag = 1; }
          ln_phase ^= 1;
          // combine the groups' (mean, M2) pairs: M2 = sum M2_g + UW * sum (mean_g - mean)^2
          float tot = 0.f;
          for (int g2 = 0; g2 < n_groups; ++g2) tot += stats[stat_slot + g2 * 32];
          const float mean = tot / (float)n_groups;
          float m2 = 0.f;
          for (int g2 = 0; g2 < n_groups; ++g2) {
            const float dm = stats[stat_slot + g2 * 32] - mean;
            m2 += stats[kEpiWarps * 32 + stat_slot + g2 * 32] + (float)UW * dm * dm;
          }
          const float rstd = rsqrtf(m2 / (float)p.N + p.eps);
          // z is staged beside y when the tile leaves room (32-column units use half of the
          // warp's staging tile); otherwise the store of y must first finish reading it
          unsigned char* zbuf = buf + (UW == 32 ? kStagingTile / 2 : 0);
          if (UW != 32) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
          }
#pragma unroll
          for (int j = 0; j < UW; j += 8) {
            const float4 gA = *reinterpret_cast<const float4*>(my_bias + 64 + j);
            const float4 gB = *reinterpret_cast<const float4*>(my_bias + 64 + j + 4);
            const float4 tA = *reinterpret_cast<const float4*>(my_bias + 128 + j);
            const float4 tB = *reinterpret_cast<const float4*>(my_bias + 128 + j + 4);
            const float g8[8] = {gA.x, gA.y, gA.z, gA.w, gB.x, gB.y, gB.z, gB.w};
            const float t8[8] = {tA.x, tA.y, tA.z, tA.w, tB.x, tB.y, tB.z, tB.w};
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
              const float2 f = unpack2<T>(yreg[(j + e) >> 1]);
              o[e >> 1] = pack2<T>(fmaf((f.x - mean) * rstd, g8[e], t8[e]), fmaf((f.y - mean) * rstd, g8[e + 1], t8[e + 1]));
            }
            *reinterpret_cast<uint4*>(zbuf + lane * RB + (((j >> 3) ^ ((lane / RPW) % CPR)) << 4)) =
                make_uint4(o[0], o[1], o[2], o[3]);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&map_z, zbuf, col0, row0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
#ifdef DCNB200_LINEAR_PROFILE
    if (blockIdx.x == 0 && warp == 2 && lane == 0)
      for (int i = 5; i < 10; ++i) g_lin_prof[i] = prof_acc[i];
#endif
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side ---------------------------------------------------------------------------

struct LinearArgs {
  int dtype;
  const void* x; const void* w; const void* residual; void* y; void* z;
};

template <typename T, int BN, int ACT>
cudaError_t launch_act(const LinearArgs& a, LinearParams p, int sms, cudaStream_t stream) {
  static std::once_flag once[64];
  static cudaError_t attr_err[64];
  int dev = 0;
  cudaGetDevice(&dev);
  dev = dev < 0 || dev >= 64 ? 0 : dev;
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(linear_kernel<T, BN, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_bytes<T, BN, ACT>());
  });
  if (attr_err[dev] != cudaSuccess) return attr_err[dev];
  CUtensorMap mx, mw, my, mr, mz;
  constexpr int UW = unit_cols<BN>();
  if (!make_map(&mx, a.dtype, a.x, p.M, p.K, kBM, kBK) || !make_map(&mw, a.dtype, a.w, p.N, p.K, BN, kBK) ||
      !make_map(&my, a.dtype, a.y, p.M, p.n_split > 0 ? p.n_split : p.N, 32, UW) ||
      !make_map(&mr, a.dtype, a.residual ? a.residual : a.y, p.M, p.n_split > 0 ? p.n_split : p.N, 32, UW) ||
      !make_map(&mz, a.dtype, a.z ? a.z : a.y, p.M, p.n_split > 0 ? p.N - p.n_split : p.N, 32, UW))
    return cudaErrorNotSupported;
  p.n_tiles = (p.N + BN - 1) / BN;
  const long long tiles = (long long)p.m_tiles * p.n_tiles;
  const int grid = (int)(tiles < sms ? tiles : sms);
  // Programmatic dependent launch pays where a launch is short (its prologue -- barriers, tensor-memory
  // allocation, GELU table -- is then a visible share of it): FlashInternImage-T at batch 32 runs 7 %
  // faster with it.  Long launches measured 1 % slower with it at batch 256, so they start the ordinary way.
  constexpr long long kPdlMaxTilesPerSm = 8;
  return launch_overlapped_if(tiles <= kPdlMaxTilesPerSm * sms, linear_kernel<T, BN, ACT>, dim3((unsigned)grid), dim3(kGemmThreads),
                              smem_bytes<T, BN, ACT>(), stream, mx, mw, my, mr, mz, p);
}

template <typename T>
cudaError_t launch_bn(int bn, int act, const LinearArgs& a, const LinearParams& p, int sms, cudaStream_t stream) {
  if (act == 2) {
    if (bn == 256) return launch_act<T, 256, 2>(a, p, sms, stream);
    if (bn == 128) return launch_act<T, 128, 2>(a, p, sms, stream);
    return launch_act<T, 64, 2>(a, p, sms, stream);
  }
  if (act == 1) {
    if (bn == 256) return launch_act<T, 256, 1>(a, p, sms, stream);
    if (bn == 128) return launch_act<T, 128, 1>(a, p, sms, stream);
    return launch_act<T, 64, 1>(a, p, sms, stream);
  }
  if (bn == 256) return launch_act<T, 256, 0>(a, p, sms, stream);
  if (bn == 128) return launch_act<T, 128, 0>(a, p, sms, stream);
  return launch_act<T, 64, 0>(a, p, sms, stream);
}

}  // namespace

// dtype: 1 fp16, 2 bf16.  Returns cudaErrorNotSupported when the driver lacks tensor maps.
// act 2 (LayerNorm as second output z; N <= 256) needs gamma, beta, eps and z.  With act 0 and
// n_split > 0 (a multiple of 64) the columns [n_split, N) are written to z as an (M, N - n_split) tensor
// and y is (M, n_split): two Linear layers over the same input in one product.
cudaError_t launch_linear_fwd(int dtype, const void* x, const void* w, const void* bias, const void* residual,
                              void* y, long long M, int N, int K, int act, int sms, int* status,
                              cudaStream_t stream, const void* gamma, const void* beta, float eps, void* z, int n_split) {
  // Tile width: the widest of 256/128/64 that N fills, unless a narrower one wastes less of the
  // last wave of CTAs (cost model: waves x (columns + fixed per-tile overhead)).
  const int m_tiles = (int)((M + kBM - 1) / kBM);
  int bn = 64;
  double best = 1e30;
  for (int cand = 256; cand >= 64; cand /= 2) {
    if (cand > 64 && N <= cand / 2) continue;
    // a ring too shallow to cover the TMA latency of a multi-block K loop is not worth the width
    const int depth = cand == 256 ? (act ? stages<__half, 256, 1>() : stages<__half, 256, 0>())
                                  : (cand == 128 ? (act ? stages<__half, 128, 1>() : stages<__half, 128, 0>()) : 8);
    if (cand > 64 && depth < 3 && (K + kBK - 1) / kBK > depth) continue;
    const long long tiles = (long long)m_tiles * ((N + cand - 1) / cand);
    const double cost = (double)((tiles + sms - 1) / sms) * (cand + 96);  // 96: fitted per-tile overhead
    if (cost < best * 0.98) { best = cost; bn = cand; }
  }
  if (act == 2) bn = N > 128 ? 256 : (N > 64 ? 128 : 64);  // a row must lie in one tile
  LinearParams p;
  p.M = M; p.N = N; p.K = K;
  p.m_tiles = (int)((M + kBM - 1) / kBM);
  p.n_tiles = 0;
  p.k_blocks = (K + kBK - 1) / kBK;
  p.bias = bias; p.residual = residual; p.y = y; p.status = status;
  p.gamma = gamma; p.beta = beta; p.eps = eps; p.n_split = n_split;
  const LinearArgs a{dtype, x, w, residual, y, z};
  if (dtype == 1) return launch_bn<__half>(bn, act, a, p, sms, stream);
  return launch_bn<__nv_bfloat16>(bn, act, a, p, sms, stream);
}

}  // namespace dcnb200

#ifdef DCNB200_LINEAR_PROFILE
extern "C" int dcnv4b200_linear_profile(long long* out16) {
  return (int)cudaMemcpyFromSymbol(out16, dcnb200::g_lin_prof, sizeof(long long) * 16);
}
#endif
