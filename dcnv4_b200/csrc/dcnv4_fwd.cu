// DCNv4 forward: out[b,y,x,g,:] = sum_k mask_k * bilinear(value[b,:,:,g,:], h_k, w_k).
//
// Replaces the reference's forward_kernel_dcn_reg + launcher
// (DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:142-325) and the zero-filled output of its host
// wrapper (DCNv4_op/src/cuda/dcnv4_cuda.cu:62): every output element is written exactly
// once, so no memset is needed.
//
// Work decomposition: persistent CTAs loop over th x tw tiles of output positions (a compact
// 2-D patch of one image, so the input pixels its samples touch stay resident in this SM's
// L1).  A tile's packed offset/mask rows -- one contiguous span per tile row -- are staged to
// shared memory with bulk copies, double-buffered so the next tile's rows arrive while the
// current tile is computed.  Work items (query, group, channel vector) are laid out
// channel-fastest so a warp's output store covers consecutive bytes.  A lane owns 32 bytes of
// channels (V is a template parameter; 16- and 64-byte lanes exist for other group sizes).
#include "common.cuh"

namespace dcnb200 {

size_t dcnv4_fwd_smem(const DcnParams& p, int elem) {
  size_t b = 16 + 2 * (size_t)p.th * p.tw * p.Ppad * elem;
  if (p.softmax) b += (size_t)p.th * p.tw * p.G * sizeof(float2);
  return b;
}

// PLAIN: 3x3 kernel without remove_center / softmax and one channel chunk per lane -- the
// configuration every FlashInternImage layer uses; everything else takes the generic path.
template <typename T, int V, bool PLAIN>
__global__ void __launch_bounds__(kThreads, DCNB200_FWD_MINB)
dcnv4_fwd_kernel(const T* __restrict__ value, const T* __restrict__ om, T* __restrict__ out,
                 const DcnParams p, int* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw);  // bar[0], bar[1]
  const size_t tbytes = (size_t)p.th * p.tw * p.Ppad * sizeof(T);
  T* s_buf[2] = {reinterpret_cast<T*>(smem_raw + 16), reinterpret_cast<T*>(smem_raw + 16 + tbytes)};
  float2* s_stat = reinterpret_cast<float2*>(smem_raw + 16 + 2 * tbytes);

  const int tiles_per_img = p.tiles_x * p.tiles_y;
  const int n_tiles = p.N * tiles_per_img;
  const int kh = PLAIN ? 3 : p.kh, kw = PLAIN ? 3 : p.kw;
  const int K = PLAIN ? 9 : p.K;
  const bool rc = PLAIN ? false : (p.remove_center != 0);
  const bool softmax = PLAIN ? false : (p.softmax != 0);
  const int chunks = PLAIN ? 1 : p.chunks;

  // tile index -> staging descriptor, issued by thread 0
  auto issue = [&](int tile, int buf) {
    const int b = tile / tiles_per_img;
    const int t_in = tile - b * tiles_per_img;
    const int tyi = t_in / p.tiles_x;
    const int y0 = tyi * p.th, x0 = (t_in - tyi * p.tiles_x) * p.tw;
    const int rows = min(p.th, p.Ho - y0), cols = min(p.tw, p.Wo - x0);
    const size_t q_first = ((size_t)b * p.Ho + y0) * p.Wo + x0;
    issue_stage(s_buf[buf], om + q_first * p.Ppad, (uint32_t)(cols * p.Ppad * sizeof(T)), rows,
                (size_t)p.Wo * p.Ppad * sizeof(T), (uint32_t)(p.tw * p.Ppad * sizeof(T)), &bar[buf]);
  };

  if (threadIdx.x == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
  }
  __syncthreads();
  // Tile order.  16-bit tensors: a contiguous share per CTA (consecutive tiles are spatial
  // neighbours, so the halo pixels they share are still in this SM's L1; shares differ by at most
  // one tile).  fp32 tensors: round-robin -- twice the bytes per pixel leave little of a neighbour
  // tile in L1 anyway, and with all CTAs inside the same few images the gathers that miss L1 hit
  // L2 (measured: 121 -> 111 us at 64x56x56x64 fp32, no change for fp16).
  constexpr bool kRoundRobin = sizeof(T) == 4;
  const int share = n_tiles / (int)gridDim.x, extra = n_tiles % (int)gridDim.x;
  const int tile_begin = kRoundRobin ? (int)blockIdx.x : (int)blockIdx.x * share + min((int)blockIdx.x, extra);
  const int tile_end = kRoundRobin ? n_tiles : tile_begin + share + ((int)blockIdx.x < extra ? 1 : 0);
  const int tile_step = kRoundRobin ? (int)gridDim.x : 1;
  pdl_trigger();
  pdl_wait();  // value and offset_mask are the previous kernels' outputs
  if (threadIdx.x == 0 && tile_begin < tile_end) issue(tile_begin, 0);

  const int cw = (p.dw * (kw - 1)) >> 1, ch = (p.dh * (kh - 1)) >> 1;
  const int center = (kw / 2) * kh + (kh / 2);
  const int n_items = p.th * p.tw * p.G * p.tpg;
  const int tpg_shift = 31 - __clz(p.tpg);
  const float dwf = (float)p.dw, dhf = (float)p.dh;
  const float Hf = (float)p.H, Wf = (float)p.W;

  int it = 0;
  for (int tile = tile_begin; tile < tile_end; tile += tile_step, ++it) {
    const int cur = it & 1;
    const int next = tile + tile_step;
    if (threadIdx.x == 0 && next < tile_end) issue(next, cur ^ 1);

    const int b = tile / tiles_per_img;
    const int t_in = tile - b * tiles_per_img;
    const int tyi = t_in / p.tiles_x;
    const int y0 = tyi * p.th, x0 = (t_in - tyi * p.tiles_x) * p.tw;
    const int rows = min(p.th, p.Ho - y0), cols = min(p.tw, p.Wo - x0);
    const T* s_om = s_buf[cur];
    wait_stage(&bar[cur], (uint32_t)((it >> 1) & 1), status);

    if (softmax) {  // per pair: max and 1/sum(exp) of the K mask logits
      for (int pr = threadIdx.x; pr < p.th * p.tw * p.G; pr += kThreads) {
        const int ql = pr / p.G;
        if (ql / p.tw < rows && ql % p.tw < cols) {
          const T* row = s_om + ql * p.Ppad + (pr % p.G) * 3 * K + 2 * K;
          float mx = -INFINITY;
          for (int k = 0; k < K; ++k) mx = fmaxf(mx, to_f32(row[k]));
          float sum = 0.f;
          for (int k = 0; k < K; ++k) sum += __expf(to_f32(row[k]) - mx);
          s_stat[pr] = make_float2(mx, 1.f / sum);
        }
      }
      __syncthreads();
    }

    const T* img_b = value + (size_t)b * p.H * p.W * p.C;
    for (int item = threadIdx.x; item < n_items; item += kThreads) {
      const int c = item & (p.tpg - 1);
      const int pr = item >> tpg_shift;
      const int ql = fast_div(pr, p.div_g);
      const int g = pr - ql * p.G;
      const int ty = fast_div(ql, p.div_tw), tx = ql - ty * p.tw;
      if (ty >= rows || tx >= cols) continue;
      const int y = y0 + ty, x = x0 + tx;

      const T* row = s_om + ql * p.Ppad + g * 3 * K;
      const float base_w = dcn_base(cw - p.pw + x * p.sw, cw, p.scale);
      const float base_h = dcn_base(ch - p.ph + y * p.sh, ch, p.scale);
      float2 stat = make_float2(0.f, 1.f);
      if (softmax) stat = s_stat[pr];
      T* out_q = out + (((size_t)b * p.Ho + y) * p.Wo + x) * p.C + g * p.D;

      for (int ci = 0; ci < chunks; ++ci) {
        const int ch0 = (c + ci * p.tpg) * V;
        const T* img = img_b + g * p.D + ch0;
        float acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = 0.f;

        if (PLAIN) {
#pragma unroll
          for (int i = 0; i < 3; ++i) {
#pragma unroll
            for (int j = 0; j < 3; ++j) {
              const int k = i * 3 + j;
              const float w_im = dcn_coord(base_w, (float)i * dwf, to_f32(row[2 * k]), p.scale);
              const float h_im = dcn_coord(base_h, (float)j * dhf, to_f32(row[2 * k + 1]), p.scale);
              fwd_point<T, V>(img, p.H, p.W, p.C, Hf, Wf, h_im, w_im, to_f32(row[18 + k]), acc);
            }
          }
        } else {
          int k = 0;
          for (int i = 0; i < kw; ++i) {
            for (int j = 0; j < kh; ++j) {
              if (rc && i * kh + j == center) continue;
              const float w_im = dcn_coord(base_w, (float)(i * p.dw), to_f32(row[2 * k]), p.scale);
              const float h_im = dcn_coord(base_h, (float)(j * p.dh), to_f32(row[2 * k + 1]), p.scale);
              float m = to_f32(row[2 * K + k]);
              if (softmax) m = __expf(m - stat.x) * stat.y;
              fwd_point<T, V>(img, p.H, p.W, p.C, Hf, Wf, h_im, w_im, m, acc);
              ++k;
            }
          }
        }
        constexpr int WORDS = V * (int)sizeof(T) / 4;
        uint32_t packed[WORDS];
        narrow(acc, packed, (const T*)nullptr);
        if constexpr (WORDS == 16) {
          uint32_t lo[8], hi[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) { lo[e] = packed[e]; hi[e] = packed[8 + e]; }
          stg_raw(out_q + ch0, lo);
          stg_raw(out_q + ch0 + V / 2, hi);
        } else {
          stg_raw(out_q + ch0, packed);
        }
      }
    }
    __syncthreads();  // all reads of this buffer are done before the copy for tile it+2 may refill it
  }
}

template <typename T, int V>
static cudaError_t launch_v(const T* value, const T* om, T* out, const DcnParams& p, int* status, cudaStream_t s) {
  const size_t smem = dcnv4_fwd_smem(p, sizeof(T));
  const bool plain = p.kh == 3 && p.kw == 3 && !p.remove_center && !p.softmax && p.chunks == 1;
  int per_sm = 1;
  cudaError_t e = plain ? persistent_ctas_per_sm<dcnv4_fwd_kernel<T, V, true>>(smem, &per_sm)
                        : persistent_ctas_per_sm<dcnv4_fwd_kernel<T, V, false>>(smem, &per_sm);
  if (e != cudaSuccess) return e;
  auto kern = plain ? dcnv4_fwd_kernel<T, V, true> : dcnv4_fwd_kernel<T, V, false>;
  const long long n_tiles = (long long)p.N * p.tiles_x * p.tiles_y;
  const long long want = (long long)p.sm_count * per_sm;
  const int grid = (int)(n_tiles < want ? n_tiles : want);
  if (plain) prefer_carveout<dcnv4_fwd_kernel<T, V, true>>((size_t)per_sm * (smem + 1024));
  else prefer_carveout<dcnv4_fwd_kernel<T, V, false>>((size_t)per_sm * (smem + 1024));
  return launch_overlapped(kern, dim3((unsigned)grid), dim3(kThreads), smem, s, value, om, out, p, status);
}

template <typename T>
static cudaError_t launch_t(const T* value, const T* om, T* out, const DcnParams& p, int* status, cudaStream_t s) {
  const int bytes = p.lane_ch * (int)sizeof(T);
  if constexpr (sizeof(T) == 4) {
    if (bytes == 64) return launch_v<T, 16>(value, om, out, p, status, s);
  }
  if (bytes == 32) return launch_v<T, 32 / (int)sizeof(T)>(value, om, out, p, status, s);
  return launch_v<T, 16 / (int)sizeof(T)>(value, om, out, p, status, s);
}

cudaError_t launch_dcnv4_fwd(int dtype, const void* value, const void* om, void* out,
                             const DcnParams& p, int* status, cudaStream_t s) {
  if (tiled_override() == 1 && dcnv4_fwd_tiled_applies(p)) {
    const cudaError_t e = launch_dcnv4_fwd_tiled(dtype, value, om, out, p, status, s);
    if (e != cudaErrorNotSupported) return e;  // no tensor-map support in the driver: other kernel
  }
  switch (dtype) {
    case 0: return launch_t((const float*)value, (const float*)om, (float*)out, p, status, s);
    case 1: return launch_t((const __half*)value, (const __half*)om, (__half*)out, p, status, s);
    default: return launch_t((const __nv_bfloat16*)value, (const __nv_bfloat16*)om, (__nv_bfloat16*)out, p, status, s);
  }
}

}  // namespace dcnb200
