// DCNv4 forward that produces its own offset/mask rows (16-bit tensors, 3x3 / stride 1 / pad 1 /
// dilation 1, 16 channels per group -- the configuration of every FlashInternImage layer):
//
//     offset_mask[q, :] = x[q, :] . W^T + bias            (the module's `offset_mask` Linear)
//     out[q, g, :]      = sum_k mask_k * bilinear(value[b, :, :, g, :], h_k, w_k)
//
// In the reference these are two steps with the (N, H, W, ceil(27 G / 8) * 8) offset/mask tensor
// written to and read back from HBM between them (DCNv4_op/DCNv4/modules/dcnv4.py:121-140 calling
// DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:142-325); that tensor is the largest one the sampling
// kernel reads.  Here the rows of 128 consecutive queries are computed on the tensor cores inside the
// CTA that samples for them and never leave the SM.
//
// A task is 128 consecutive queries x 4 groups (the last task of a query tile has fewer when the group
// count is not a multiple of 4).  The 27 columns of a group (nine (dx, dy) pairs, then nine masks)
// occupy a slot of 32 accumulator columns: the rows of W that belong to a group are loaded as a 32-row
// box of their own, so a task's product is 128 x 128 and every group starts on a 32-column boundary of
// tensor memory.  One persistent CTA per SM, eighteen warps:
//   warp 0     producer : TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle, this GPU's memory, no
//                         multicast) of the x tile (128 x 64) and of four boxes of W (32 x 64 each) into
//                         a shared-memory ring, one slot per 64 input features;
//   warp 1     MMA      : one lane issues tcgen05.mma (M = 128, N = 128, K = 16, fp32 accumulate)
//                         into one of two accumulators in tensor memory, so the product of task i+1
//                         runs while task i is being sampled;
//   warps 2-17 workers  : four independent teams of four warps, one team per quadrant of tensor memory
//                         (tensor memory hands the lanes of warp w rows 32 (w % 4) .. + 31 of the
//                         accumulator, i.e. 32 of the task's queries).  Each warp of a team reads the
//                         32-column slots of every fourth group (tcgen05.ld), adds the bias, rounds to
//                         the storage type -- exactly what the Linear would have written -- and parks
//                         the 27 values per (query, group) in the team's part of a shared-memory
//                         stage, then releases the accumulator.  After a barrier among
//                         the team's 128 threads every lane takes (query, group) pairs, group fastest --
//                         the lanes of a warp then sample around few distinct pixels, which is what the
//                         L1 gather rate rewards -- and samples as the stand-alone forward kernel does:
//                         one 32-byte load per bilinear corner, fp32 arithmetic, one 32-byte store of
//                         the 16 output channels.  The offset/mask rows never reach global memory.
// Every mbarrier wait is bounded.  A worker warp whose wait runs out records kStatusStageTimeout and
// raises its team's flag; the flag is only ever written before the first of a task's two team barriers
// and read right after it, so the team leaves the loop together and no warp is left waiting at a
// barrier.  The producer and the MMA lane stop on their own bounded waits, and the CTA frees its tensor
// memory.
#include <mutex>

#include "gelu_table.cuh"
#include "tc.cuh"

namespace dcnb200 {

namespace {

using namespace tc;

constexpr int kQ = 128;           // queries per task == rows of the product == tensor-memory lanes
constexpr int kBK = 64;           // input features per ring slot: 128 bytes == one swizzle span
constexpr int kUmmaK = 16;
constexpr int kWorkWarps = 16;
constexpr int kWorkThreads = 32 * kWorkWarps;
constexpr int kFusedThreads = 64 + kWorkThreads;
constexpr int kPts = 27;          // offset/mask columns of one group: 9 x (dx, dy), then 9 masks

constexpr int kSlot = 32;         // accumulator columns (and rows of a W box) per group
constexpr uint32_t kBoxBytes = kSlot * kBK * 2;

template <int GC> constexpr int acc_cols() { return GC * kSlot; }  // 128, 256
// At most two ring slots and a single parking area keep the CTA below 100 KB of shared memory: the sampling
// phase lives on L1 hits (the gathers of neighbouring queries overlap), and shared memory is carved
// out of the same 256 KB as L1.  Measured at 64 x 56 x 56 x 64 fp16: L1 hit rate 63 % with 190 KB of
// shared memory against 91 % for the stand-alone kernel with 57 KB.
// A single 64-feature block per task needs one slot only (the two accumulators already let the loads
// and the product of the next task run ahead); deeper reductions alternate between two.
inline int ring_stages(int k_blocks) { return k_blocks == 1 ? 1 : 2; }
constexpr int kGroupBytes = 56;   // 27 parked 16-bit values of one (query, group), padded to 8 bytes
// Row pitch of the parked rows: 16 bytes more than the groups need, so that the 16-byte stores of eight
// neighbouring lanes (eight queries) fall into eight different bank groups.
template <int GC> constexpr int row_pitch() { return GC * kGroupBytes + 16; }
template <int GC> constexpr uint32_t slot_bytes() { return (uint32_t)(kQ * kBK * 2 + acc_cols<GC>() * kBK * 2); }
constexpr int kBarrierBytes = 256;

struct FusedParams {
  long long M;       // N * H * W queries
  int H, W, G, C;    // C = 16 G
  int k_blocks, m_tiles, chunks;
  int stages;        // ring slots
  int n_cols;        // 27 G: columns of the Linear that carry offsets and masks
  int bias_floats;   // staged bias: 28 floats per group (27 + one of padding, for 16-byte loads)
  float scale;
  const void* bias;  // (>= n_cols) or null
  int* status;
};

template <int GC>
size_t fused_smem(int bias_floats, int stages) {
  return 1024 + (size_t)stages * slot_bytes<GC>() + (size_t)kQ * row_pitch<GC>() +
         (size_t)bias_floats * 4 + kBarrierBytes;
}

__device__ __forceinline__ void work_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kWorkThreads) : "memory"); }
// barrier among the four warps of a quadrant team (ids 2..5)
__device__ __forceinline__ void team_barrier(int quad) { asm volatile("bar.sync %0, 128;" ::"r"(quad + 2) : "memory"); }

template <typename T, int GC>
__global__ void __launch_bounds__(kFusedThreads, 1)
dcnv4_fwd_fused_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                       const T* __restrict__ value, T* __restrict__ out, const FusedParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int BN = acc_cols<GC>(), PITCH = row_pitch<GC>();
  const int kStages = p.stages;
  constexpr uint32_t kBytesA = kQ * kBK * 2, kBytesB = BN * kBK * 2;
  unsigned char* ring_a = smem;
  unsigned char* ring_b = smem + kStages * kBytesA;
  unsigned char* s_om = ring_b + kStages * kBytesB;  // [kQ] parked rows
  float* s_bias = reinterpret_cast<float*>(s_om + kQ * PITCH);
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_bias + p.bias_floats);
  uint64_t* full = bars;                         // [kStages] TMA landed
  uint64_t* empty = bars + kStages;              // [kStages] MMA finished reading
  uint64_t* acc_full = bars + 2 * kStages;       // [2] accumulator complete
  uint64_t* acc_empty = bars + 2 * kStages + 2;  // [2] accumulator read by every worker warp
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);  // producer / MMA gave up
  volatile int* team_abort = abort_flag + 1;  // [4 teams] a warp of the team gave up

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = 2 * BN;  // 256 or 512

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], kWorkWarps); }
    *abort_flag = 0;
    for (int i = 0; i < 4; ++i) team_abort[i] = 0;
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
  pdl_wait();  // x and value are earlier kernels' outputs; out may still be read by one

  // Each CTA takes a contiguous share of the tasks (shares differ by at most one): consecutive tasks are
  // the next groups of the same queries and then the next 128 queries, about two image rows further down,
  // whose samples fall on rows this SM's L1 still holds.
  const long long n_tasks = (long long)p.m_tiles * p.chunks;
  const long long share = n_tasks / gridDim.x, extra = n_tasks % gridDim.x;
  const long long t_begin = blockIdx.x * share + (blockIdx.x < extra ? blockIdx.x : extra);
  const long long t_end = t_begin + share + (blockIdx.x < extra ? 1 : 0);

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (long long t = t_begin; t < t_end && !*abort_flag; ++t) {
        const int mt = (int)(t / p.chunks), ch = (int)(t - (long long)mt * p.chunks);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_bounded(&empty[stage], phase ^ 1)) { atomicExch(p.status, kStatusStageTimeout); *abort_flag = 1; break; }
          mbar_expect_tx(&full[stage], kBytesA + kBytesB);
          tma_load_2d(ring_a + stage * kBytesA, &map_x, kb * kBK, mt * kQ, &full[stage]);
          // rows 27 g .. 27 g + 31 of W for each group of the task; the last five rows of a box
          // belong to the next group (or lie beyond W and read as zero) and feed columns nobody reads
#pragma unroll
          for (int j = 0; j < GC; ++j)
            tma_load_2d(ring_b + stage * kBytesB + j * kBoxBytes, &map_w, kb * kBK, (ch * GC + j) * kPts, &full[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc<T>(BN, kQ);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (long long t = t_begin; t < t_end && !*abort_flag; ++t) {
        if (!mbar_wait_bounded(&acc_empty[acc], acc_phase ^ 1)) { atomicExch(p.status, kStatusStageTimeout); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_bounded(&full[stage], phase)) { atomicExch(p.status, kStatusStageTimeout); *abort_flag = 1; break; }
          tc_fence_after();
          const uint64_t da = smem_desc_sw128(ring_a + stage * kBytesA);
          const uint64_t db = smem_desc_sw128(ring_b + stage * kBytesB);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            tc_mma_f16(d_tmem, da + (uint64_t)(k * kUmmaK * 2 / 16), db + (uint64_t)(k * kUmmaK * 2 / 16), idesc,
                       (kb | k) != 0);
          tc_commit(&empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        tc_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- workers
    const int wtid = (int)threadIdx.x - 64;
    const int quad = warp & 3;          // tensor-memory lanes [32 quad, 32 quad + 32): the team's queries
    const int member = (warp - 2) >> 2;  // 0..3 within the team
    const int tl = member * 32 + lane;   // 0..127 within the team
    constexpr int kSlots = GC / 4;       // group slots a warp parks per task
    {
      const T* bias = static_cast<const T*>(p.bias);
      for (int i = wtid; i < p.bias_floats; i += kWorkThreads) {
        const int g = i / 28, c = i - g * 28;
        s_bias[i] = (bias != nullptr && c < kPts && g < p.G) ? to_f32(bias[g * kPts + c]) : 0.f;
      }
    }
    work_barrier();

    const int HW = p.H * p.W;
    const float Hf = (float)p.H, Wf = (float)p.W;
    // n / d as umulhi(n, floor(2^32 / d) + 1): never below the quotient and at most one above it for
    // n < 2^31, which one comparison repairs.
    const uint32_t mul_hw = (uint32_t)(0x100000000ull / (uint32_t)HW) + 1u;
    const uint32_t mul_w = (uint32_t)(0x100000000ull / (uint32_t)p.W) + 1u;
    uint32_t it = 0;
    for (long long t = t_begin; t < t_end; ++t, ++it) {
      const int acc = (int)(it & 1);
      const uint32_t acc_phase = (it >> 1) & 1;
      const int mt = (int)(t / p.chunks), ch = (int)(t - (long long)mt * p.chunks);
      unsigned char* stage_rows = s_om + (size_t)(quad * 32) * PITCH;
      const bool landed = mbar_wait_bounded(&acc_full[acc], acc_phase);
      if (!landed && lane == 0) { atomicExch(p.status, kStatusStageTimeout); team_abort[quad] = 1; }
      if (landed) {  // warp-uniform
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < kSlots; ++j) {
          const int gl = member + 4 * j;
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + gl * kSlot), v);
          tmem_ld_wait();
          const float4* b4 = reinterpret_cast<const float4*>(s_bias + (ch * GC + gl) * 28);
          uint32_t o[14];
#pragma unroll
          for (int i = 0; i < 7; ++i) {  // the 28th value (padding) is parked too and never read
            const float4 b = b4[i];
            o[2 * i] = pack2<T>(__uint_as_float(v[4 * i]) + b.x, __uint_as_float(v[4 * i + 1]) + b.y);
            o[2 * i + 1] = pack2<T>(__uint_as_float(v[4 * i + 2]) + b.z, __uint_as_float(v[4 * i + 3]) + b.w);
          }
          unsigned char* dst = stage_rows + lane * PITCH + gl * kGroupBytes;  // 8-byte aligned
#pragma unroll
          for (int i = 0; i < 14; i += 2) *reinterpret_cast<uint2*>(dst + i * 4) = make_uint2(o[i], o[i + 1]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      team_barrier(quad);  // the team's rows of this task are parked
      if (team_abort[quad]) break;

#pragma unroll 1
      for (int item = tl; item < 32 * GC; item += 128) {
        const int ql = item / GC, gl = item % GC;
        const int q = mt * kQ + quad * 32 + ql;  // M < 2^31 - 128 (checked by the caller)
        if (q >= (int)p.M || ch * GC + gl >= p.G) continue;
        int b = HW == 1 ? q : (int)__umulhi((uint32_t)q, mul_hw);
        int r = q - b * HW;
        if (r < 0) { --b; r += HW; }
        int y = p.W == 1 ? r : (int)__umulhi((uint32_t)r, mul_w);
        int x = r - y * p.W;
        if (x < 0) { --y; x += p.W; }
        // the 27 parked values of this (query, group): seven 8-byte loads
        uint32_t omw[14];
        {
          const uint2* src = reinterpret_cast<const uint2*>(stage_rows + ql * PITCH + gl * kGroupBytes);
#pragma unroll
          for (int i = 0; i < 7; ++i) { const uint2 u = src[i]; omw[2 * i] = u.x; omw[2 * i + 1] = u.y; }
        }
        // 3x3 / stride 1 / pad 1 / dilation 1: first tap at (x - 1, y - 1) before scaling
        const float base_w = dcn_base(x, 1, p.scale);
        const float base_h = dcn_base(y, 1, p.scale);
        const int g = ch * GC + gl;
        const T* img = value + (size_t)b * HW * p.C + g * 16;
        float a16[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) a16[e] = 0.f;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            const int k = i * 3 + j;
            const float2 off = unpack2<T>(omw[k]);  // (dx, dy) of tap k
            const float2 mk = unpack2<T>(omw[(18 + k) >> 1]);
            const float w_im = dcn_coord(base_w, (float)i, off.x, p.scale);
            const float h_im = dcn_coord(base_h, (float)j, off.y, p.scale);
            fwd_point<T, 16>(img, p.H, p.W, p.C, Hf, Wf, h_im, w_im, ((18 + k) & 1) ? mk.y : mk.x, a16);
          }
        }
        uint32_t packed[8];
        narrow(a16, packed, (const T*)nullptr);
        stg_raw(out + (size_t)q * p.C + g * 16, packed);
      }
      team_barrier(quad);  // every parked row has been read: the next task may overwrite them
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, int GC>
cudaError_t launch_gc(int dtype, const void* value, const void* x, const void* w, void* out, FusedParams p, int w_rows,
                      int K, int sms, cudaStream_t stream) {
  p.chunks = (p.G + GC - 1) / GC;  // a ragged last task computes columns of groups that do not exist
  p.bias_floats = 28 * GC * p.chunks;
  p.stages = ring_stages(p.k_blocks);
  const size_t smem = fused_smem<GC>(p.bias_floats, p.stages);
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];
  int dev = 0;
  cudaGetDevice(&dev);
  dev = dev < 0 || dev >= 64 ? 0 : dev;
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(dcnv4_fwd_fused_kernel<T, GC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024);
  });
  if (attr_err[dev] != cudaSuccess) return attr_err[dev];
  CUtensorMap mx, mw;
  if (!make_map(&mx, dtype, x, p.M, K, kQ, kBK) || !make_map(&mw, dtype, w, w_rows, K, kSlot, kBK))
    return cudaErrorNotSupported;
  const long long tasks = (long long)p.m_tiles * p.chunks;
  const int grid = (int)(tasks < sms ? tasks : sms);
  prefer_carveout<dcnv4_fwd_fused_kernel<T, GC>>(smem + 1024);
  return launch_overlapped(dcnv4_fwd_fused_kernel<T, GC>, dim3((unsigned)grid), dim3(kFusedThreads), smem, stream, mx,
                           mw, static_cast<const T*>(value), static_cast<T*>(out), p);
}

}  // namespace

bool dcnv4_fwd_fused_applies(int dtype, int G, int D, int K, int w_rows) {
  return (dtype == 1 || dtype == 2) && D == 16 && G > 0 && K > 0 && K % 8 == 0 &&
         w_rows >= kPts * G && G <= 128;
}

// value (N,H,W,16 G), x (N*H*W, K), w (w_rows, K) with w_rows >= 27 G, bias (w_rows) or null, out like
// value; dtype 1 fp16, 2 bf16.  Returns cudaErrorNotSupported when the driver lacks tensor maps.
cudaError_t launch_dcnv4_fwd_fused(int dtype, const void* value, const void* x, const void* w, const void* bias,
                                   void* out, int N, int H, int W, int G, int K, int w_rows, float scale, int sms,
                                   int* status, cudaStream_t stream) {
  FusedParams p;
  p.M = (long long)N * H * W;
  p.H = H; p.W = W; p.G = G; p.C = 16 * G;
  p.k_blocks = (K + kBK - 1) / kBK;
  p.m_tiles = (int)((p.M + kQ - 1) / kQ);
  p.chunks = 0;
  p.stages = 0;
  p.n_cols = kPts * G;
  p.bias_floats = 0;
  p.scale = scale;
  p.bias = bias;
  p.status = status;
  if (dtype == 1) return launch_gc<__half, 4>(dtype, value, x, w, out, p, w_rows, K, sms, stream);
  return launch_gc<__nv_bfloat16, 4>(dtype, value, x, w, out, p, w_rows, K, sms, stream);
}

}  // namespace dcnb200
