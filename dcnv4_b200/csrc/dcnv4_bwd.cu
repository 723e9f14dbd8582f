// DCNv4 backward: grad_value (scatter) and grad_offset_mask (per-point reductions).
//
// Replaces backward_kernel_dcn_warp_primitive / backward_kernel_dcn and their launcher
// (DCNv4_op/src/cuda/dcnv4_col2im_cuda.cuh:20-472, helper DCNv4_op/src/cuda/common.h:100-212)
// plus the zero-fills and the fp16 cast passes of the host wrapper
// (DCNv4_op/src/cuda/dcnv4_cuda.cu:133-139,169-174).
//
//  * A lane owns 4 channels of a pair (V is a template parameter; 8 is also instantiated).  Its
//    grad_value contribution to a bilinear corner is one 16-byte vector reduction
//    (red.global.add.v4.f32) into the fp32 accumulation buffer, and the lanes of a pair cover
//    the corner's contiguous bytes in one instruction.
//  * The three per-point partials (d/dx, d/dy, d/dmask) are reduced over the lanes of a pair
//    with warp shuffles.  Lane 0 of the pair deposits them in a shared-memory image of the
//    tile's grad_offset_mask rows; the CTA then writes whole rows (pad columns included, as
//    zeros) with coalesced 16-byte stores, so grad_offset_mask needs no memset.
//  * 2-D query tiles and double-buffered bulk-copy staging as in the forward kernel; persistent
//    CTAs when there are few tiles, one CTA per tile when there are thousands (see launch_v).
#include <cstdlib>

#include "common.cuh"

namespace dcnb200 {

size_t dcnv4_bwd_smem(const DcnParams& p, int elem) {
  const size_t q = (size_t)p.th * p.tw;
  size_t b = 16 + 2 * q * p.Ppad * elem + q * p.Ppad * sizeof(float);
  if (p.softmax) b += q * p.G * sizeof(float2);
  return b;
}

template <typename T, int V, bool PLAIN>
__global__ void __launch_bounds__(kThreads, DCNB200_BWD_MINB)
dcnv4_bwd_kernel(const T* __restrict__ value, const T* __restrict__ om, const T* __restrict__ gout,
                 float* __restrict__ gvalue, T* __restrict__ gom, const DcnParams p, int* status) {
  constexpr int VS = 16 / (int)sizeof(T);  // elements per 16-byte store of the write-out
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw);
  const int n_q = p.th * p.tw;
  const size_t tbytes = (size_t)n_q * p.Ppad * sizeof(T);
  T* s_buf[2] = {reinterpret_cast<T*>(smem_raw + 16), reinterpret_cast<T*>(smem_raw + 16 + tbytes)};
  float* s_g = reinterpret_cast<float*>(smem_raw + 16 + 2 * tbytes);
  float2* s_stat = reinterpret_cast<float2*>(s_g + (size_t)n_q * p.Ppad);

  const int tiles_per_img = p.tiles_x * p.tiles_y;
  const int n_tiles = p.N * tiles_per_img;
  const int kh = PLAIN ? 3 : p.kh, kw = PLAIN ? 3 : p.kw;
  const int K = PLAIN ? 9 : p.K;
  const bool rc = PLAIN ? false : (p.remove_center != 0);
  const bool softmax = PLAIN ? false : (p.softmax != 0);
  const int chunks = PLAIN ? 1 : p.chunks_b;
  const int used = 3 * K * p.G;

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
  // pad columns of the gradient rows are zeros; lanes never write them, so once is enough
  for (int i = threadIdx.x; i < n_q * (p.Ppad - used); i += kThreads)
    s_g[(i / (p.Ppad - used)) * p.Ppad + used + i % (p.Ppad - used)] = 0.f;
  __syncthreads();
  // this CTA's contiguous share of the tiles (consecutive tiles are spatial neighbours, so
  // the halo pixels they share are still in this SM's L1); shares differ by at most one tile
  const int share = n_tiles / (int)gridDim.x, extra = n_tiles % (int)gridDim.x;
  const int tile_begin = (int)blockIdx.x * share + min((int)blockIdx.x, extra);
  const int tile_end = tile_begin + share + ((int)blockIdx.x < extra ? 1 : 0);
  if (threadIdx.x == 0 && tile_begin < tile_end) issue(tile_begin, 0);

  const int cw = (p.dw * (kw - 1)) >> 1, ch = (p.dh * (kh - 1)) >> 1;
  const int center = (kw / 2) * kh + (kh / 2);
  const int tpg = p.tpg_b;
  const int tpg_shift = 31 - __clz(tpg);
  const int n_items = n_q * p.G * tpg;
  const float dwf = (float)p.dw, dhf = (float)p.dh;
  const float Hf = (float)p.H, Wf = (float)p.W;

  int it = 0;
  for (int tile = tile_begin; tile < tile_end; ++tile, ++it) {
    const int cur = it & 1;
    const int next = tile + 1;
    if (threadIdx.x == 0 && next < tile_end) issue(next, cur ^ 1);

    const int b = tile / tiles_per_img;
    const int t_in = tile - b * tiles_per_img;
    const int tyi = t_in / p.tiles_x;
    const int y0 = tyi * p.th, x0 = (t_in - tyi * p.tiles_x) * p.tw;
    const int rows = min(p.th, p.Ho - y0), cols = min(p.tw, p.Wo - x0);
    const size_t q_first = ((size_t)b * p.Ho + y0) * p.Wo + x0;
    const T* s_om = s_buf[cur];
    wait_stage(&bar[cur], (uint32_t)((it >> 1) & 1), status);

    if (softmax) {
      for (int pr = threadIdx.x; pr < n_q * p.G; pr += kThreads) {
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

    const size_t img_b = (size_t)b * p.H * p.W * p.C;
    // Every lane of a warp takes part in the shuffles, so the loop runs over whole CTA-wide
    // strides; lanes without a valid query work on query 0 with all memory traffic disabled.
    for (int base = 0; base < n_items; base += kThreads) {
      const int item = base + threadIdx.x;
      const int c = item & (tpg - 1);
      const int pr_raw = item >> tpg_shift;
      const int ql_raw = fast_div(pr_raw, p.div_g);
      const int ty_raw = fast_div(ql_raw, p.div_tw), tx_raw = ql_raw - ty_raw * p.tw;
      const bool active = item < n_items && ty_raw < rows && tx_raw < cols;
      const int ql = active ? ql_raw : 0;
      const int g = active ? pr_raw - ql_raw * p.G : 0;
      const int ty = active ? ty_raw : 0, tx = active ? tx_raw : 0;
      const int y = y0 + ty, x = x0 + tx;

      const T* row = s_om + ql * p.Ppad + g * 3 * K;
      float* grow = s_g + ql * p.Ppad + g * 3 * K;
      const float base_w = dcn_base(cw - p.pw + x * p.sw, cw, p.scale);
      const float base_h = dcn_base(ch - p.ph + y * p.sh, ch, p.scale);
      float2 stat = make_float2(0.f, 1.f);
      if (softmax) stat = s_stat[ql * p.G + g];

      const T* img = value + img_b + g * p.D + c * V;
      float* gimg = gvalue + img_b + g * p.D + c * V;
      const T* go_ptr = gout + (((size_t)b * p.Ho + y) * p.Wo + x) * p.C + g * p.D + c * V;
      float gy0[V];
      gather_corner<T, V>(go_ptr, active, gy0);

      if (PLAIN) {
#pragma unroll
        for (int i = 0; i < 3; ++i) {
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            const int k = i * 3 + j;
            const float w_im = dcn_coord(base_w, (float)i * dwf, to_f32(row[2 * k]), p.scale);
            const float h_im = dcn_coord(base_h, (float)j * dhf, to_f32(row[2 * k + 1]), p.scale);
            const float m = to_f32(row[18 + k]);
            float gx = 0.f, gyv = 0.f, gm = 0.f;
            const bool ok = bwd_point<T, V>(img, gimg, p.H, p.W, p.C, Hf, Wf, h_im, w_im, m, active, gy0,
                                            gx, gyv, gm);
            for (int o = tpg >> 1; o > 0; o >>= 1) {
              gx += __shfl_xor_sync(0xffffffffu, gx, o);
              gyv += __shfl_xor_sync(0xffffffffu, gyv, o);
              gm += __shfl_xor_sync(0xffffffffu, gm, o);
            }
            if (active && c == 0) {
              const float sm = p.scale * m;
              grow[2 * k] = ok ? sm * gx : 0.f;
              grow[2 * k + 1] = ok ? sm * gyv : 0.f;
              grow[18 + k] = ok ? gm : 0.f;
            }
          }
        }
      } else {
        float soft_sum = 0.f;  // sum_k t_k (softmax backward), kept by lane 0 of the pair
        int k = 0;
        for (int i = 0; i < kw; ++i) {
          for (int j = 0; j < kh; ++j) {
            if (rc && i * kh + j == center) continue;
            const float w_im = dcn_coord(base_w, (float)(i * p.dw), to_f32(row[2 * k]), p.scale);
            const float h_im = dcn_coord(base_h, (float)(j * p.dh), to_f32(row[2 * k + 1]), p.scale);
            float m = to_f32(row[2 * K + k]);
            if (softmax) m = __expf(m - stat.x) * stat.y;
            float gx = 0.f, gyv = 0.f, gm = 0.f;
            bool ok = bwd_point<T, V>(img, gimg, p.H, p.W, p.C, Hf, Wf, h_im, w_im, m, active, gy0, gx, gyv, gm);
            for (int ci = 1; ci < chunks; ++ci) {
              const int off = ci * tpg * V;
              float gy[V];
              gather_corner<T, V>(go_ptr + off, active, gy);
              ok = bwd_point<T, V>(img + off, gimg + off, p.H, p.W, p.C, Hf, Wf, h_im, w_im, m, active, gy,
                                   gx, gyv, gm);
            }
            for (int o = tpg >> 1; o > 0; o >>= 1) {
              gx += __shfl_xor_sync(0xffffffffu, gx, o);
              gyv += __shfl_xor_sync(0xffffffffu, gyv, o);
              gm += __shfl_xor_sync(0xffffffffu, gm, o);
            }
            if (active && c == 0) {
              const float sm = p.scale * m;
              grow[2 * k] = ok ? sm * gx : 0.f;
              grow[2 * k + 1] = ok ? sm * gyv : 0.f;
              const float gmk = ok ? gm : 0.f;
              if (softmax) {
                grow[2 * K + k] = gmk * m;
                soft_sum += gmk * m;
              } else {
                grow[2 * K + k] = gmk;
              }
            }
            ++k;
          }
        }
        if (softmax && active && c == 0) {
          for (int t = 0; t < K; ++t) {
            const float m = __expf(to_f32(row[2 * K + t]) - stat.x) * stat.y;
            grow[2 * K + t] -= m * soft_sum;
          }
        }
      }
    }

    __syncthreads();
    // coalesced write-out of the tile's grad_offset_mask rows (one contiguous span per tile row)
    const int vec_per_row = cols * p.Ppad / VS;
    for (int i = threadIdx.x; i < rows * vec_per_row; i += kThreads) {
      const int r = i / vec_per_row, j = i - r * vec_per_row;
      const float* src = s_g + (size_t)r * p.tw * p.Ppad + (size_t)j * VS;
      float v[VS];
#pragma unroll
      for (int e = 0; e < VS; e += 4) {
        const float4 f4 = *reinterpret_cast<const float4*>(src + e);
        v[e] = f4.x; v[e + 1] = f4.y; v[e + 2] = f4.z; v[e + 3] = f4.w;
      }
      uint32_t packed[4];
      narrow(v, packed, (const T*)nullptr);
      stg_raw(gom + (q_first + (size_t)r * p.Wo) * p.Ppad + (size_t)j * VS, packed);
    }
    __syncthreads();  // s_g and this staging buffer are free for the next tile
  }
}

template <typename T, int V>
static cudaError_t launch_v(const T* value, const T* om, const T* gout, float* gvalue, T* gom,
                            const DcnParams& p, int* status, cudaStream_t s) {
  const size_t smem = dcnv4_bwd_smem(p, sizeof(T));
  const bool plain = p.kh == 3 && p.kw == 3 && !p.remove_center && !p.softmax && p.chunks_b == 1;
  int per_sm = 1;
  cudaError_t e = plain ? persistent_ctas_per_sm<dcnv4_bwd_kernel<T, V, true>>(smem, &per_sm)
                        : persistent_ctas_per_sm<dcnv4_bwd_kernel<T, V, false>>(smem, &per_sm);
  if (e != cudaSuccess) return e;
  auto kern = plain ? dcnv4_bwd_kernel<T, V, true> : dcnv4_bwd_kernel<T, V, false>;
  const long long n_tiles = (long long)p.N * p.tiles_x * p.tiles_y;
  const long long want = (long long)p.sm_count * per_sm;
  // Measured on B200: with thousands of tiles the reduction-bound backward runs ~10 % faster
  // when every tile is its own short-lived CTA (their phases de-synchronise naturally); with
  // few tiles per SM the persistent, double-buffered form wins.
  const int grid = (int)((n_tiles < want || n_tiles >= 4 * want) ? n_tiles : want);
  kern<<<grid, kThreads, smem, s>>>(value, om, gout, gvalue, gom, p, status);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_t(const T* value, const T* om, const T* gout, float* gvalue, T* gom,
                            const DcnParams& p, int* status, cudaStream_t s) {
  return p.lane_ch_b == 8 ? launch_v<T, 8>(value, om, gout, gvalue, gom, p, status, s)
                          : launch_v<T, 4>(value, om, gout, gvalue, gom, p, status, s);
}

int tiled_override() {
  const char* e = getenv("DCNV4B200_TILED");
  return (e && (e[0] == '0' || e[0] == '1') && e[1] == 0) ? e[0] - '0' : -1;
}

cudaError_t launch_dcnv4_bwd(int dtype, const void* value, const void* om, const void* gout,
                             float* gvalue_f32, void* gom, const DcnParams& p, int* status, cudaStream_t s) {
  // The shared-memory pre-accumulating kernel (dcnv4_bwd_tiled.cu) is correct but measured about
  // twice as slow as this one on B200 at every tile size tried, so it is never chosen
  // automatically; DCNV4B200_TILED=1 selects it for the configurations it covers.
  if (tiled_override() == 1 && dcnv4_bwd_tiled_applies(p)) {
    const cudaError_t e = launch_dcnv4_bwd_tiled(dtype, value, om, gout, gvalue_f32, gom, p, status, s);
    if (e != cudaErrorNotSupported) return e;  // no tensor-map support in the driver: other kernel
  }
  switch (dtype) {
    case 0: return launch_t((const float*)value, (const float*)om, (const float*)gout, gvalue_f32, (float*)gom, p, status, s);
    case 1: return launch_t((const __half*)value, (const __half*)om, (const __half*)gout, gvalue_f32, (__half*)gom, p, status, s);
    default: return launch_t((const __nv_bfloat16*)value, (const __nv_bfloat16*)om, (const __nv_bfloat16*)gout, gvalue_f32, (__nv_bfloat16*)gom, p, status, s);
  }
}

}  // namespace dcnb200
