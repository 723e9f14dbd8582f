// extern "C" boundary: argument validation, launch geometry, dispatch.  See
// include/dcnv4_b200.h for the contract of every entry point and the reference interface
// each one replaces.
#include "../../include/dcnv4_b200.h"

#include <mutex>

#include "common.cuh"

using namespace dcnb200;

namespace {

// One status word per device; kernels that give up on a bounded wait record it here.
__device__ int g_status_word;

constexpr int kMaxDevices = 64;
std::mutex g_mu;
int* g_status_ptr[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};

// Status word address and SM count of the current device (looked up once per device).
int status_ptr(int** out, int* sm_count = nullptr) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return DCNV4B200_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_status_word);
    if (e != cudaSuccess) return (int)e;
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    g_sm_count[dev] = sms > 0 ? sms : 1;
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  *out = g_status_ptr[dev];
  if (sm_count) *sm_count = g_sm_count[dev];
  return 0;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }
inline int elem_size(int dtype) { return dtype == DCNV4B200_F32 ? 4 : 2; }
inline bool dtype_ok(int dtype) { return dtype >= DCNV4B200_F32 && dtype <= DCNV4B200_BF16; }

// D == per_lane * tpg * chunks with tpg the largest power of two (<= 32) dividing D/per_lane.
void split_lanes(int D, int per_lane, int* tpg, int* chunks) {
  const int nvec = D / per_lane;
  int t = 1;
  while (t < 32 && nvec % (t * 2) == 0) t *= 2;
  *tpg = t;
  *chunks = nvec / t;
}

FastDiv make_div(int d) {
  FastDiv f;
  f.d = (uint32_t)d;
  f.mul = d > 1 ? (uint32_t)(0x100000000ULL / (uint64_t)d) + 1u : 0u;
  return f;
}

// Lane geometry of a pair, chosen from measurements on B200 (random 64-byte gathers): the L1
// serves about one distinct 128-byte line per cycle whatever the access width, so a
// bilinear corner of a pair should be fetched by ONE load instruction -- lanes * vector bytes
// == group bytes -- and a pair's vector reductions should likewise share one instruction.
//  * forward lane: 32 bytes of channels (one 256-bit load per corner) when D*elem is a multiple
//    of 32 and the tensors are 32-byte aligned, else 16 bytes;
//  * backward lane: 4 channels, i.e. exactly one red.global.add.v4.f32 per corner.
// D*elem must be a multiple of 16.
#ifndef DCNB200_FWD_LANE_BYTES
#define DCNB200_FWD_LANE_BYTES 32
#endif
#ifndef DCNB200_BWD_LANE_CH
#define DCNB200_BWD_LANE_CH 4
#endif
#ifndef DCNB200_TILES_PER_SM
#define DCNB200_TILES_PER_SM 6
#endif
#ifndef DCNB200_MIN_PASSES
#define DCNB200_MIN_PASSES 1
#endif
template <typename P>
int lane_geometry(P& p, int D, int dtype, bool wide_fwd, bool wide_bwd) {
  const int es = elem_size(dtype);
  if (D <= 0 || (D * es) % 16 != 0) return DCNV4B200_ERR_CHANNELS;
  int lane = 16 / es;
  for (int cand = DCNB200_FWD_LANE_BYTES / es; cand * es > 16; cand /= 2)
    if (D % cand == 0 && wide_fwd) { lane = cand; break; }
  p.lane_ch = lane;
  split_lanes(D, lane, &p.tpg, &p.chunks);
  p.lane_ch_b = (DCNB200_BWD_LANE_CH == 8 && D % 8 == 0 && (es == 2 || wide_bwd)) ? 8 : 4;
  split_lanes(D, p.lane_ch_b, &p.tpg_b, &p.chunks_b);
  return 0;
}

// 2-D query tile of one CTA for the DCNv4 kernels: at most `max_q` queries (what fits the
// shared-memory budget, capped so that a CTA keeps a few items per thread), as square as the
// divisors of the output size allow, and small enough to leave several tiles per SM.
void pick_tile_2d(int N, int Ho, int Wo, size_t bytes_per_query, int items_per_query, int sm_count, int* th, int* tw) {
  // The search below is pure arithmetic on its arguments; a small per-thread memo keeps it off
  // the per-call path of a training loop that repeats the same few shapes.
  struct Memo { int N, Ho, Wo, ipq, sms; size_t bpq; int th, tw; };
  constexpr int kMemo = 16;
  thread_local Memo memo[kMemo] = {};
  thread_local int memo_next = 0;
  for (int i = 0; i < kMemo; ++i) {
    const Memo& m = memo[i];
    if (m.th && m.N == N && m.Ho == Ho && m.Wo == Wo && m.ipq == items_per_query && m.sms == sm_count &&
        m.bpq == bytes_per_query) {
      *th = m.th; *tw = m.tw;
      return;
    }
  }
  struct Save {
    Memo* slot; int* th; int* tw;
    ~Save() { slot->th = *th; slot->tw = *tw; }
  } save{&memo[memo_next], th, tw};
  memo[memo_next] = Memo{N, Ho, Wo, items_per_query, sm_count, bytes_per_query, 0, 0};
  memo_next = (memo_next + 1) % kMemo;
  long long max_q = (long long)((kSmemBudget - 64) / bytes_per_query);  // 64: barriers + alignment slack
  const long long cap_items = (6LL * kThreads + items_per_query - 1) / items_per_query;
  if (max_q > cap_items) max_q = cap_items;
  // Several tiles per SM -- but a tile never shrinks below DCNB200_MIN_PASSES full passes of
  // the CTA's threads: on a small batch idle lanes cost more than idle SMs.
  long long cap_grid = (long long)N * Ho * Wo / ((long long)sm_count * DCNB200_TILES_PER_SM);
  const long long min_q = ((long long)DCNB200_MIN_PASSES * kThreads + items_per_query - 1) / items_per_query;
  if (cap_grid < min_q) cap_grid = min_q;
  if (max_q > cap_grid) max_q = cap_grid;
  if (max_q < 1) max_q = 1;
  // Score every shape that fits: the fraction of lane slots doing useful work (items of a tile
  // are processed in passes of kThreads), the fraction of the tile grid that lies inside the
  // image (ragged edges), and a mild preference for compact, larger tiles (L1 locality).
  double best = -1.0;
  int bh = 1, bw = 1;
  const int h_max = Ho < kMaxTileRows ? Ho : kMaxTileRows;
  const int w_max = Wo < 64 ? Wo : 64;
  for (int h = 1; h <= h_max; ++h) {
    for (int w = 1; w <= w_max && (long long)h * w <= max_q; ++w) {
      const long long items = (long long)h * w * items_per_query;
      const long long passes = (items + kThreads - 1) / kThreads;
      const double lane_eff = (double)items / (double)(passes * kThreads);
      const long long covered = (long long)((Ho + h - 1) / h) * h * ((Wo + w - 1) / w) * w;
      const double edge_eff = (double)Ho * Wo / (double)covered;
      const int thin = h < w ? h : w;
      const double compact = 1.0 - 0.5 / (double)thin;
      const double size_bonus = 1.0 - 1.0 / (double)(4 + h * w);
      const double score = lane_eff * edge_eff * compact * size_bonus;
      if (score > best + 1e-9) { best = score; bh = h; bw = w; }
    }
  }
  *th = bh;
  *tw = bw;
}

// Queries per CTA of the 1-D tiles (FlashDeformAttn): as many as fit the staging budget, but
// never so many that the grid drops below a few CTAs per SM; `unit` keeps every tile start
// 16-byte aligned.
int pick_tile(long long nq, size_t bytes_per_query, int unit, int items_per_query, int sm_count) {
  long long t = (long long)((kSmemBudget - 128) / bytes_per_query);
  const long long cap_items = (6LL * kThreads + items_per_query - 1) / items_per_query;
  if (t > cap_items) t = cap_items;
  const long long cap_grid = nq / ((long long)sm_count * DCNB200_TILES_PER_SM);
  if (cap_grid >= 1 && t > cap_grid) t = cap_grid;
  if (t > 128) t = 128;
  t = (t / unit) * unit;
  if (t < unit) t = unit;
  return (int)t;
}

int fill_dcn(DcnParams& p, int dtype, int N, int H, int W, int G, int D, int kh, int kw, int sh, int sw,
             int ph, int pw, int dh, int dw, float offset_scale, int remove_center, int Ppad, int softmax,
             bool backward, bool wide_fwd = false, bool wide_bwd = false) {
  if (!dtype_ok(dtype)) return DCNV4B200_ERR_DTYPE;
  if (N <= 0 || H <= 0 || W <= 0 || G <= 0 || D <= 0 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 ||
      ph < 0 || pw < 0 || dh <= 0 || dw <= 0)
    return DCNV4B200_ERR_SHAPE;
  const int Ho = dcnv4b200_out_size(H, ph, dh, kh, sh), Wo = dcnv4b200_out_size(W, pw, dw, kw, sw);
  if (Ho <= 0 || Wo <= 0) return DCNV4B200_ERR_SHAPE;
  const int K = kh * kw - (remove_center ? 1 : 0);
  if (K <= 0) return DCNV4B200_ERR_SHAPE;
  if (Ppad % 8 != 0 || (long long)Ppad < 3LL * K * G) return DCNV4B200_ERR_PADDED_DIM;
  if (int rc = lane_geometry(p, D, dtype, wide_fwd, wide_bwd)) return rc;
  const long long nq = (long long)N * Ho * Wo;
  if (nq >= (1LL << 31) || (long long)H * W * G * D >= (1LL << 31) || (long long)G * D >= (1 << 24))
    return DCNV4B200_ERR_TOO_LARGE;
  // shared memory per query: two staging buffers, the fp32 gradient rows (backward), softmax stats
  const size_t bpq = 2 * (size_t)Ppad * elem_size(dtype) + (backward ? (size_t)Ppad * 4 : 0) +
                     (softmax ? (size_t)G * 8 : 0);
  if (bpq + 64 > (size_t)kSmemBudget) return DCNV4B200_ERR_UNSUPPORTED;
  p.N = N; p.H = H; p.W = W; p.G = G; p.D = D; p.C = G * D; p.Ho = Ho; p.Wo = Wo;
  p.kh = kh; p.kw = kw; p.sh = sh; p.sw = sw; p.ph = ph; p.pw = pw; p.dh = dh; p.dw = dw;
  p.K = K; p.Ppad = Ppad; p.remove_center = remove_center ? 1 : 0; p.softmax = softmax ? 1 : 0;
  p.scale = offset_scale;
  p.nq = (int)nq;
  p.div_g = make_div(G);
  p.th = p.tw = p.tiles_x = p.tiles_y = 0;  // chosen by tile_dcn() once the device is known
  p.sm_count = 0;
  return 0;
}

// Query tile of the validated problem `p` for a device with `sm_count` SMs (arguments are checked
// before the device is touched, so this runs as a second step).
int tile_dcn(DcnParams& p, int dtype, bool backward, int sm_count) {
  if (sm_count < 1) sm_count = 1;
  const size_t bpq = 2 * (size_t)p.Ppad * elem_size(dtype) + (backward ? (size_t)p.Ppad * 4 : 0) +
                     (p.softmax ? (size_t)p.G * 8 : 0);
  pick_tile_2d(p.N, p.Ho, p.Wo, bpq, p.G * (backward ? p.tpg_b : p.tpg), sm_count, &p.th, &p.tw);
  p.tiles_x = (p.Wo + p.tw - 1) / p.tw;
  p.tiles_y = (p.Ho + p.th - 1) / p.th;
  if ((long long)p.N * p.tiles_x * p.tiles_y >= (1LL << 31)) return DCNV4B200_ERR_TOO_LARGE;
  p.div_tw = make_div(p.tw);
  p.sm_count = sm_count;
  return 0;
}

int fill_fda(FdaParams& p, int dtype, int B, int Len_in, int G, int D, int L, int Len_q, int K, bool backward,
             bool wide_fwd = false, bool wide_bwd = false) {
  if (!dtype_ok(dtype)) return DCNV4B200_ERR_DTYPE;
  if (B <= 0 || Len_in <= 0 || G <= 0 || D <= 0 || L <= 0 || Len_q <= 0 || K <= 0) return DCNV4B200_ERR_SHAPE;
  if (L > kMaxLevels) return DCNV4B200_ERR_UNSUPPORTED;
  if (int rc = lane_geometry(p, D, dtype, wide_fwd, wide_bwd)) return rc;
  const long long nq = (long long)B * Len_q;
  if (nq >= (1LL << 31) || (long long)Len_in * G * D >= (1LL << 31) || (long long)G * D >= (1 << 24))
    return DCNV4B200_ERR_TOO_LARGE;
  const int es = elem_size(dtype);
  const size_t row_bytes = (size_t)G * 3 * L * K * es;
  // smallest number of queries whose rows span a multiple of 16 bytes
  int unit = 1;
  while ((row_bytes * unit) % 16 != 0) unit *= 2;
  const size_t bpq = 2 * row_bytes + (backward ? (size_t)G * 3 * L * K * 4 : 0) + (size_t)G * 8;
  if (bpq * unit + 128 > (size_t)kSmemBudget) return DCNV4B200_ERR_UNSUPPORTED;
  p.B = B; p.Len_in = Len_in; p.G = G; p.D = D; p.C = G * D; p.L = L; p.Len_q = Len_q; p.K = K; p.LK = L * K;
  p.nq = (int)nq;
  p.tile = unit;  // chosen by tile_fda() once the device is known
  p.div_g = make_div(G);
  p.sm_count = 0;
  return 0;
}

int tile_fda(FdaParams& p, int dtype, bool backward, int sm_count) {
  if (sm_count < 1) sm_count = 1;
  const int es = elem_size(dtype);
  const size_t row_bytes = (size_t)p.G * 3 * p.L * p.K * es;
  int unit = 1;
  while ((row_bytes * unit) % 16 != 0) unit *= 2;
  const size_t bpq = 2 * row_bytes + (backward ? (size_t)p.G * 3 * p.L * p.K * 4 : 0) + (size_t)p.G * 8;
  p.tile = pick_tile(p.nq, bpq, unit, p.G * (backward ? p.tpg_b : p.tpg), sm_count);
  while ((size_t)p.tile * bpq + 128 > (size_t)kSmemBudget && p.tile > unit) p.tile -= unit;
  p.sm_count = sm_count;
  return 0;
}

}  // namespace

extern "C" {

int dcnv4b200_abi_version(void) { return DCNV4B200_ABI_VERSION; }

const char* dcnv4b200_strerror(int code) {
  switch (code) {
    case DCNV4B200_OK: return "success";
    case DCNV4B200_ERR_NULL: return "a required pointer is NULL";
    case DCNV4B200_ERR_DTYPE: return "unknown dtype code (0 fp32, 1 fp16, 2 bf16)";
    case DCNV4B200_ERR_SHAPE: return "non-positive or inconsistent dimension";
    case DCNV4B200_ERR_ALIGN: return "pointer not 16-byte aligned";
    case DCNV4B200_ERR_WORKSPACE: return "workspace missing or smaller than *_bwd_workspace_bytes()";
    case DCNV4B200_ERR_UNSUPPORTED:
      return "outside the supported parameter space (more than 8 levels, or one query's packed row "
             "exceeds the shared-memory staging budget)";
    case DCNV4B200_ERR_PADDED_DIM: return "padded_offset_dim must be a multiple of 8 and >= 3*K*group";
    case DCNV4B200_ERR_CHANNELS: return "group_channels must be a multiple of 4 (fp32) or 8 (fp16/bf16)";
    case DCNV4B200_ERR_TOO_LARGE: return "tensor too large for 31-bit indexing";
    case DCNV4B200_ERR_SCRATCH_LIMIT:
      return "N*H*W*G*D exceeds the built-in scratch of dcnv4b200_bwd_static_scratch "
             "(see dcnv4b200_bwd_static_scratch_max_elements); use dcnv4b200_bwd with a workspace";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "unknown error code";
}

int dcnv4b200_out_size(int in, int pad, int dil, int k, int stride) {
  if (stride <= 0) return 0;
  const int span = in + 2 * pad - (dil * (k - 1) + 1);
  if (span < 0) return 0;
  return span / stride + 1;
}

int dcnv4b200_fwd(const void* value, const void* offset_mask, void* out, int dtype, int N, int H, int W,
                  int G, int D, int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                  float offset_scale, int remove_center, int padded_offset_dim, int softmax, void* stream) {
  if (!value || !offset_mask || !out) return DCNV4B200_ERR_NULL;
  if (!aligned16(value) || !aligned16(offset_mask) || !aligned16(out)) return DCNV4B200_ERR_ALIGN;
  DcnParams p;
  if (int rc = fill_dcn(p, dtype, N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw, offset_scale, remove_center,
                        padded_offset_dim, softmax, false, aligned32(value) && aligned32(out)))
    return rc;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  if (int rc = tile_dcn(p, dtype, false, sms)) return rc;
  return (int)launch_dcnv4_fwd(dtype, value, offset_mask, out, p, status, static_cast<cudaStream_t>(stream));
}

size_t dcnv4b200_bwd_workspace_bytes(int dtype, int N, int H, int W, int G, int D) {
  if (dtype == DCNV4B200_F32 || !dtype_ok(dtype) || N <= 0 || H <= 0 || W <= 0 || G <= 0 || D <= 0) return 0;
  return (size_t)N * H * W * G * D * sizeof(float);
}

int dcnv4b200_bwd(const void* value, const void* offset_mask, const void* grad_out, void* grad_value,
                  void* grad_offset_mask, void* workspace, size_t workspace_bytes, int dtype, int N, int H,
                  int W, int G, int D, int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                  float offset_scale, int remove_center, int padded_offset_dim, int softmax, void* stream) {
  if (!value || !offset_mask || !grad_out || !grad_value || !grad_offset_mask) return DCNV4B200_ERR_NULL;
  if (!aligned16(value) || !aligned16(offset_mask) || !aligned16(grad_out) || !aligned16(grad_value) ||
      !aligned16(grad_offset_mask) || !aligned16(workspace))
    return DCNV4B200_ERR_ALIGN;
  DcnParams p;
  if (int rc = fill_dcn(p, dtype, N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw, offset_scale, remove_center,
                        padded_offset_dim, softmax, true, false, aligned32(value) && aligned32(grad_out)))
    return rc;
  const size_t need = dcnv4b200_bwd_workspace_bytes(dtype, N, H, W, G, D);
  if (need && (!workspace || workspace_bytes < need)) return DCNV4B200_ERR_WORKSPACE;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  if (int rc = tile_dcn(p, dtype, true, sms)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t n = (size_t)N * H * W * G * D;
  float* acc = need ? static_cast<float*>(workspace) : static_cast<float*>(grad_value);
  cudaError_t e = cudaMemsetAsync(acc, 0, n * sizeof(float), s);
  if (e != cudaSuccess) return (int)e;
  e = launch_dcnv4_bwd(dtype, value, offset_mask, grad_out, acc, grad_offset_mask, p, status, s);
  if (e != cudaSuccess) return (int)e;
  if (need) e = launch_convert_f32(dtype, acc, grad_value, n, sms, s);
  return (int)e;
}

int fdab200_fwd(const void* value, const int64_t* spatial_shapes, const int64_t* level_start_index,
                const void* sampling_loc_attn, void* out, int dtype, int B, int Len_in, int G, int D, int L,
                int Len_q, int K, void* stream) {
  if (!value || !spatial_shapes || !level_start_index || !sampling_loc_attn || !out) return DCNV4B200_ERR_NULL;
  if (!aligned16(value) || !aligned16(sampling_loc_attn) || !aligned16(out)) return DCNV4B200_ERR_ALIGN;
  FdaParams p;
  if (int rc = fill_fda(p, dtype, B, Len_in, G, D, L, Len_q, K, false, aligned32(value) && aligned32(out)))
    return rc;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  tile_fda(p, dtype, false, sms);
  return (int)launch_fda_fwd(dtype, value, spatial_shapes, level_start_index, sampling_loc_attn, out, p, status,
                             static_cast<cudaStream_t>(stream));
}

size_t fdab200_bwd_workspace_bytes(int dtype, int B, int Len_in, int G, int D) {
  if (dtype == DCNV4B200_F32 || !dtype_ok(dtype) || B <= 0 || Len_in <= 0 || G <= 0 || D <= 0) return 0;
  return (size_t)B * Len_in * G * D * sizeof(float);
}

int fdab200_bwd(const void* value, const int64_t* spatial_shapes, const int64_t* level_start_index,
                const void* sampling_loc_attn, const void* grad_out, void* grad_value,
                void* grad_sampling_loc_attn, void* workspace, size_t workspace_bytes, int dtype, int B,
                int Len_in, int G, int D, int L, int Len_q, int K, void* stream) {
  if (!value || !spatial_shapes || !level_start_index || !sampling_loc_attn || !grad_out || !grad_value ||
      !grad_sampling_loc_attn)
    return DCNV4B200_ERR_NULL;
  if (!aligned16(value) || !aligned16(sampling_loc_attn) || !aligned16(grad_out) || !aligned16(grad_value) ||
      !aligned16(grad_sampling_loc_attn) || !aligned16(workspace))
    return DCNV4B200_ERR_ALIGN;
  FdaParams p;
  if (int rc = fill_fda(p, dtype, B, Len_in, G, D, L, Len_q, K, true, false, aligned32(value) && aligned32(grad_out)))
    return rc;
  const size_t need = fdab200_bwd_workspace_bytes(dtype, B, Len_in, G, D);
  if (need && (!workspace || workspace_bytes < need)) return DCNV4B200_ERR_WORKSPACE;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  tile_fda(p, dtype, true, sms);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t n = (size_t)B * Len_in * G * D;
  float* acc = need ? static_cast<float*>(workspace) : static_cast<float*>(grad_value);
  cudaError_t e = cudaMemsetAsync(acc, 0, n * sizeof(float), s);
  if (e != cudaSuccess) return (int)e;
  e = launch_fda_bwd(dtype, value, spatial_shapes, level_start_index, sampling_loc_attn, grad_out, acc,
                     grad_sampling_loc_attn, p, status, s);
  if (e != cudaSuccess) return (int)e;
  if (need) e = launch_convert_f32(dtype, acc, grad_value, n, sms, s);
  return (int)e;
}

int dcnv4b200_fwd_corners(const void* offset_mask, int32_t* corners, int dtype, int N, int H, int W, int G,
                          int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw, float offset_scale,
                          int remove_center, int padded_offset_dim, void* stream) {
  if (!offset_mask || !corners) return DCNV4B200_ERR_NULL;
  DcnParams p;
  const int D = 16 / elem_size(dtype);  // channel count is irrelevant to the coordinates
  if (int rc = fill_dcn(p, dtype, N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw, offset_scale, remove_center,
                        padded_offset_dim, 0, false))
    return rc;
  return (int)launch_dcnv4_corners(dtype, offset_mask, corners, p, static_cast<cudaStream_t>(stream));
}

int fdab200_fwd_corners(const int64_t* spatial_shapes, const void* sampling_loc_attn, int32_t* corners,
                        int dtype, int B, int G, int L, int Len_q, int K, void* stream) {
  if (!spatial_shapes || !sampling_loc_attn || !corners) return DCNV4B200_ERR_NULL;
  FdaParams p;
  if (int rc = fill_fda(p, dtype, B, 1, G, 16 / elem_size(dtype), L, Len_q, K, false)) return rc;
  return (int)launch_fda_corners(dtype, spatial_shapes, sampling_loc_attn, corners, p,
                                 static_cast<cudaStream_t>(stream));
}

int dcnv4b200_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, int dtype,
                            int param_dtype, long long rows, int C, float eps, void* stream) {
  return dcnv4b200_layernorm_act_fwd(x, gamma, beta, y, dtype, param_dtype, rows, C, eps, DCNV4B200_ACT_NONE, stream);
}

int dcnv4b200_layernorm_act_fwd(const void* x, const void* gamma, const void* beta, void* y, int dtype,
                                int param_dtype, long long rows, int C, float eps, int activation, void* stream) {
  if (!x || !gamma || !beta || !y) return DCNV4B200_ERR_NULL;
  if (activation != DCNV4B200_ACT_NONE && activation != DCNV4B200_ACT_GELU) return DCNV4B200_ERR_UNSUPPORTED;
  if (!dtype_ok(dtype) || (param_dtype != DCNV4B200_F32 && param_dtype != dtype)) return DCNV4B200_ERR_DTYPE;
  if (rows < 0 || C <= 0) return DCNV4B200_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(y)) return DCNV4B200_ERR_ALIGN;
  if ((C * elem_size(dtype)) % 16 != 0) return DCNV4B200_ERR_CHANNELS;
  if (C > layernorm_max_channels(dtype)) return DCNV4B200_ERR_UNSUPPORTED;
  if (rows == 0) return 0;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  return (int)launch_layernorm_fwd(dtype, param_dtype, x, gamma, beta, y, rows, C, eps, activation, sms,
                                   static_cast<cudaStream_t>(stream));
}

int dcnv4b200_center_scale_blend_fwd(const void* x, const void* x_proj, const void* weight, const void* bias,
                                     void* out, int dtype, int param_dtype, long long rows, int G, int D,
                                     void* stream) {
  if (!x || !x_proj || !weight || !bias || !out) return DCNV4B200_ERR_NULL;
  if (!dtype_ok(dtype) || (param_dtype != DCNV4B200_F32 && param_dtype != dtype)) return DCNV4B200_ERR_DTYPE;
  if (rows < 0 || G <= 0 || D <= 0) return DCNV4B200_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(x_proj) || !aligned16(out) || !aligned16(weight)) return DCNV4B200_ERR_ALIGN;
  if ((D * elem_size(dtype)) % 16 != 0) return DCNV4B200_ERR_CHANNELS;
  if ((long long)G * D > center_scale_max_channels(dtype) || G > center_scale_max_groups()) return DCNV4B200_ERR_UNSUPPORTED;
  if (rows == 0) return 0;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  return (int)launch_center_scale_blend(dtype, param_dtype, x, x_proj, weight, bias, out, rows, G, D, sms,
                                        static_cast<cudaStream_t>(stream));
}

int dcnv4b200_linear_fwd(const void* x, const void* weight, const void* bias, const void* residual, void* y,
                         int dtype, long long M, int N, int K, int activation, void* stream) {
  if (!x || !weight || !y) return DCNV4B200_ERR_NULL;
  if (dtype != DCNV4B200_F16 && dtype != DCNV4B200_BF16) return DCNV4B200_ERR_DTYPE;
  if (M < 0 || N <= 0 || K <= 0) return DCNV4B200_ERR_SHAPE;
  if (activation != DCNV4B200_ACT_NONE && activation != DCNV4B200_ACT_GELU) return DCNV4B200_ERR_UNSUPPORTED;
  if (N % 8 != 0 || K % 8 != 0) return DCNV4B200_ERR_CHANNELS;
  if (!aligned16(x) || !aligned16(weight) || !aligned16(y) || !aligned16(bias) || !aligned16(residual))
    return DCNV4B200_ERR_ALIGN;
  if (M >= (1LL << 31)) return DCNV4B200_ERR_TOO_LARGE;
  if (M == 0) return 0;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  return (int)launch_linear_fwd(dtype, x, weight, bias, residual, y, M, N, K, activation, sms, status,
                                static_cast<cudaStream_t>(stream));
}

int dcnv4b200_linear_ln_fwd(const void* x, const void* weight, const void* bias, const void* residual, void* y,
                            const void* gamma, const void* beta, float eps, void* z, int dtype, long long M,
                            int N, int K, void* stream) {
  if (!x || !weight || !y || !gamma || !beta || !z) return DCNV4B200_ERR_NULL;
  if (dtype != DCNV4B200_F16 && dtype != DCNV4B200_BF16) return DCNV4B200_ERR_DTYPE;
  if (M < 0 || N <= 0 || K <= 0) return DCNV4B200_ERR_SHAPE;
  if (N > 256) return DCNV4B200_ERR_UNSUPPORTED;  // a row has to fit one tile of the kernel
  // every epilogue warp must own a full unit of columns: 32 up to N = 128, 64 above
  if (N % (N > 128 ? 64 : 32) != 0 || K % 8 != 0) return DCNV4B200_ERR_CHANNELS;
  if (!aligned16(x) || !aligned16(weight) || !aligned16(y) || !aligned16(z) || !aligned16(bias) ||
      !aligned16(residual) || !aligned16(gamma) || !aligned16(beta))
    return DCNV4B200_ERR_ALIGN;
  if (M >= (1LL << 31)) return DCNV4B200_ERR_TOO_LARGE;
  if (M == 0) return 0;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  return (int)launch_linear_fwd(dtype, x, weight, bias, residual, y, M, N, K, 2, sms, status,
                                static_cast<cudaStream_t>(stream), gamma, beta, eps, z);
}

int dcnv4b200_linear_pair_fwd(const void* x, const void* weight, const void* bias, void* y1, int N1, void* y2,
                              int N2, int dtype, long long M, int K, void* stream) {
  if (!x || !weight || !y1 || !y2) return DCNV4B200_ERR_NULL;
  if (dtype != DCNV4B200_F16 && dtype != DCNV4B200_BF16) return DCNV4B200_ERR_DTYPE;
  if (M < 0 || N1 <= 0 || N2 <= 0 || K <= 0) return DCNV4B200_ERR_SHAPE;
  // the boundary between the two outputs must fall between two 64-column store units
  if (N1 % 64 != 0 || N2 % 8 != 0 || K % 8 != 0) return DCNV4B200_ERR_CHANNELS;
  if (!aligned16(x) || !aligned16(weight) || !aligned16(y1) || !aligned16(y2) || !aligned16(bias))
    return DCNV4B200_ERR_ALIGN;
  if (M >= (1LL << 31)) return DCNV4B200_ERR_TOO_LARGE;
  if (M == 0) return 0;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  return (int)launch_linear_fwd(dtype, x, weight, bias, nullptr, y1, M, N1 + N2, K, 0, sms, status,
                                static_cast<cudaStream_t>(stream), nullptr, nullptr, 0.f, y2, N1);
}

int dcnv4b200_fwd_fused_offset(const void* value, const void* x, const void* weight, const void* bias, void* out,
                               int dtype, int N, int H, int W, int G, int D, int K, int weight_rows,
                               float offset_scale, void* stream) {
  if (!value || !x || !weight || !out) return DCNV4B200_ERR_NULL;
  if (dtype != DCNV4B200_F16 && dtype != DCNV4B200_BF16) return DCNV4B200_ERR_DTYPE;
  if (N < 0 || H <= 0 || W <= 0 || G <= 0 || D <= 0 || K <= 0 || weight_rows <= 0) return DCNV4B200_ERR_SHAPE;
  if (weight_rows < 27 * G) return DCNV4B200_ERR_PADDED_DIM;
  if (K % 8 != 0) return DCNV4B200_ERR_CHANNELS;
  if (!dcnv4_fwd_fused_applies(dtype, G, D, K, weight_rows)) return DCNV4B200_ERR_UNSUPPORTED;
  // a lane fetches the 16 channels of a group with one 32-byte load
  if (!aligned32(value) || !aligned32(out) || !aligned16(x) || !aligned16(weight) || ((uintptr_t)bias & 1))
    return DCNV4B200_ERR_ALIGN;
  if ((long long)N * H * W >= (1LL << 31) - 128 || (long long)N * H * W * G * D >= (1LL << 31))
    return DCNV4B200_ERR_TOO_LARGE;
  if (N == 0) return 0;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  return (int)launch_dcnv4_fwd_fused(dtype, value, x, weight, bias, out, N, H, W, G, K, weight_rows, offset_scale,
                                     sms, status, static_cast<cudaStream_t>(stream));
}

int dcnv4b200_bias_act_fwd(const void* x, const void* bias, void* y, int dtype, long long rows, int C,
                           int activation, void* stream) {
  if (!x || !bias || !y) return DCNV4B200_ERR_NULL;
  if (dtype != DCNV4B200_F16 && dtype != DCNV4B200_BF16) return DCNV4B200_ERR_DTYPE;
  if (rows < 0 || C <= 0) return DCNV4B200_ERR_SHAPE;
  if (activation != DCNV4B200_ACT_NONE && activation != DCNV4B200_ACT_GELU) return DCNV4B200_ERR_UNSUPPORTED;
  if (C % 8 != 0) return DCNV4B200_ERR_CHANNELS;
  if (!aligned16(x) || !aligned16(y) || !aligned16(bias)) return DCNV4B200_ERR_ALIGN;
  if (rows == 0) return 0;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  return (int)launch_bias_act_fwd(dtype, x, bias, y, rows, C, activation, sms, static_cast<cudaStream_t>(stream));
}

int dcnv4b200_device_status(int* status_out) {
  if (!status_out) return DCNV4B200_ERR_NULL;
  int* status = nullptr;
  if (int rc = status_ptr(&status)) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  e = cudaMemcpy(status_out, status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return (int)e;
  const int zero = 0;
  e = cudaMemcpy(status, &zero, sizeof(int), cudaMemcpyHostToDevice);
  return (int)e;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Backward for callers that cannot allocate device memory.
//
// Some hosts of this library run the operator from inside an execution callback of a larger
// runtime (an inference server's or a plugin framework's "enqueue" hook, a real-time loop)
// where cudaMalloc is off limits: it synchronises the whole device, and it can simply fail
// once the host application has handed all remaining device memory to its own arena.  Such a
// caller can supply inputs and outputs, but has nowhere to get the fp32 accumulation buffer
// that the 16-bit backward needs.  For them the buffer lives inside the library image.
// (The runtime reserves the array when this module is first loaded on a device -- with lazy
// loading, at the first call of any entry point there -- so such a host calls
// dcnv4b200_device_status() once per device at start-up, before it claims the memory.)

namespace {

// fp32 accumulation scratch of the allocation-free backward.  Every GPU that loads this
// library carries these 16 MiB until the process exits, whether the entry point is used or
// not; that is why the limit is modest.
constexpr size_t kStaticScratchFloats = size_t(4) << 20;  // 4 Mi floats = 16 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address.
// The real address is looked up once per device, with that device current.
float* g_static_scratch_ptr[kMaxDevices] = {nullptr};

int static_scratch_ptr(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return DCNV4B200_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_static_scratch_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" {

size_t dcnv4b200_bwd_static_scratch_max_elements(void) { return kStaticScratchFloats; }

int dcnv4b200_bwd_static_scratch(const void* value, const void* offset_mask, const void* grad_out,
                                 void* grad_value, void* grad_offset_mask, int dtype, int N, int H, int W,
                                 int G, int D, int kh, int kw, int sh, int sw, int ph, int pw, int dh,
                                 int dw, float offset_scale, int remove_center, int padded_offset_dim,
                                 int softmax, void* stream) {
  if (!value || !offset_mask || !grad_out || !grad_value || !grad_offset_mask) return DCNV4B200_ERR_NULL;
  if (!aligned16(value) || !aligned16(offset_mask) || !aligned16(grad_out) || !aligned16(grad_value) ||
      !aligned16(grad_offset_mask))
    return DCNV4B200_ERR_ALIGN;
  DcnParams p;
  if (int rc = fill_dcn(p, dtype, N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw, offset_scale, remove_center,
                        padded_offset_dim, softmax, true, false, aligned32(value) && aligned32(grad_out)))
    return rc;
  const size_t n = (size_t)N * H * W * G * D;
  const bool needs_scratch = dtype != DCNV4B200_F32;
  if (needs_scratch && n > kStaticScratchFloats) return DCNV4B200_ERR_SCRATCH_LIMIT;
  int* status = nullptr;
  int sms = 1;
  if (int rc = status_ptr(&status, &sms)) return rc;
  if (int rc = tile_dcn(p, dtype, true, sms)) return rc;
  float* acc = static_cast<float*>(grad_value);
  if (needs_scratch) {
    if (int rc = static_scratch_ptr(&acc)) return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The scratch keeps whatever the previous call left in it: clear the part this call sums into.
  cudaError_t e = cudaMemsetAsync(acc, 0, n * sizeof(float), s);
  if (e != cudaSuccess) return (int)e;
  e = launch_dcnv4_bwd(dtype, value, offset_mask, grad_out, acc, grad_offset_mask, p, status, s);
  if (e != cudaSuccess) return (int)e;
  if (needs_scratch) e = launch_convert_f32(dtype, acc, grad_value, n, sms, s);
  return (int)e;
}

}  // extern "C"
