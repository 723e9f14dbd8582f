// DCNv4 forward: out[b,y,x,g,:] = sum_k mask_k * bilinear(value[b,:,:,g,:], h_k, w_k).
//
// Replaces the reference's forward_kernel_dcn_reg + launcher
// (DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:142-325) and the zero-filled output of its host
// wrapper (DCNv4_op/src/cuda/dcnv4_cuda.cu:62): every output element is written exactly
// once, so no memset is needed.
//
// Work decomposition: a CTA takes a th x tw tile of output positions of one image (a compact
// 2-D patch, so the input pixels its samples touch stay resident in this SM's L1).  The
// tile's packed offset/mask rows -- one contiguous span per tile row -- are staged to shared
// memory with bulk copies.  Work items (query, group, channel vector) are laid out
// channel-fastest so a warp's output store covers consecutive bytes.  A lane owns VB = 32
// bytes of channels: the sampling arithmetic of a point is done once per 16 fp16 (8 fp32)
// channels and each corner is one 256-bit load.
#include "common.cuh"

namespace dcnb200 {

size_t dcnv4_fwd_smem(const DcnParams& p, int elem) {
  size_t b = 16 + (size_t)p.th * p.tw * p.Ppad * elem;
  if (p.softmax) b += (size_t)p.th * p.tw * p.G * sizeof(float2);
  return b;
}

template <typename T, int VB, int KH, int KW>
__global__ void __launch_bounds__(kThreads, 2)
dcnv4_fwd_kernel(const T* __restrict__ value, const T* __restrict__ om, T* __restrict__ out,
                 const DcnParams p, int* status) {
  constexpr int V = VB / (int)sizeof(T);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw);
  T* s_om = reinterpret_cast<T*>(smem_raw + 16);
  float2* s_stat = reinterpret_cast<float2*>(smem_raw + 16 + (size_t)p.th * p.tw * p.Ppad * sizeof(T));

  // tile -> (image, first row, first column)
  const int tiles_per_img = p.tiles_x * p.tiles_y;
  const int b = blockIdx.x / tiles_per_img;
  const int t_in = blockIdx.x - b * tiles_per_img;
  const int y0 = (t_in / p.tiles_x) * p.th, x0 = (t_in % p.tiles_x) * p.tw;
  const int rows = min(p.th, p.Ho - y0), cols = min(p.tw, p.Wo - x0);
  const size_t q_first = ((size_t)b * p.Ho + y0) * p.Wo + x0;
  if (!stage_rows(s_om, om + q_first * p.Ppad, (uint32_t)(cols * p.Ppad * sizeof(T)), rows,
                  (size_t)p.Wo * p.Ppad * sizeof(T), (uint32_t)(p.tw * p.Ppad * sizeof(T)), bar, status))
    return;

  const int kh = KH ? KH : p.kh, kw = KW ? KW : p.kw;
  const int K = p.K;

  if (p.softmax) {  // per pair: max and 1/sum(exp) of the K mask logits
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

  const int cw = (p.dw * (kw - 1)) >> 1, ch = (p.dh * (kh - 1)) >> 1;
  const int center = (kw / 2) * kh + (kh / 2);
  const int n_items = p.th * p.tw * p.G * p.tpg;
  const T* img_b = value + (size_t)b * p.H * p.W * p.C;
  const float dwf = (float)p.dw, dhf = (float)p.dh;

  for (int item = threadIdx.x; item < n_items; item += kThreads) {
    const int c = item % p.tpg;
    const int pr = item / p.tpg;
    const int g = pr % p.G;
    const int ql = pr / p.G;
    const int ty = ql / p.tw, tx = ql - ty * p.tw;
    if (ty >= rows || tx >= cols) continue;
    const int y = y0 + ty, x = x0 + tx;

    const T* row = s_om + ql * p.Ppad + g * 3 * K;
    const float base_w = dcn_base(cw - p.pw + x * p.sw, cw, p.scale);
    const float base_h = dcn_base(ch - p.ph + y * p.sh, ch, p.scale);
    float2 stat = make_float2(0.f, 1.f);
    if (p.softmax) stat = s_stat[pr];
    T* out_q = out + (((size_t)b * p.Ho + y) * p.Wo + x) * p.C + g * p.D;

    for (int ci = 0; ci < p.chunks; ++ci) {
      const int ch0 = (c + ci * p.tpg) * V;
      const T* img = img_b + g * p.D + ch0;
      float acc[V];
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] = 0.f;

#pragma unroll
      for (int i = 0; i < kw; ++i) {
#pragma unroll
        for (int j = 0; j < kh; ++j) {
          const int t = i * kh + j;
          if (p.remove_center && t == center) continue;
          const int k = t - ((p.remove_center && t > center) ? 1 : 0);
          const float w_im = dcn_coord(base_w, (float)i * dwf, to_f32(row[2 * k]), p.scale);
          const float h_im = dcn_coord(base_h, (float)j * dhf, to_f32(row[2 * k + 1]), p.scale);
          float m = to_f32(row[2 * K + k]);
          if (p.softmax) m = __expf(m - stat.x) * stat.y;
          fwd_point<T, VB>(img, p.H, p.W, p.C, h_im, w_im, m, acc);
        }
      }
      uint32_t packed[VB / 4];
      narrow(acc, packed, (const T*)nullptr);
      stg_raw(out_q + ch0, packed);
    }
  }
}

template <typename T, int VB>
static cudaError_t launch_vb(const T* value, const T* om, T* out, const DcnParams& p, int* status, cudaStream_t s) {
  const int grid = p.N * p.tiles_x * p.tiles_y;
  const size_t smem = dcnv4_fwd_smem(p, sizeof(T));
  if (p.kh == 3 && p.kw == 3)
    dcnv4_fwd_kernel<T, VB, 3, 3><<<grid, kThreads, smem, s>>>(value, om, out, p, status);
  else
    dcnv4_fwd_kernel<T, VB, 0, 0><<<grid, kThreads, smem, s>>>(value, om, out, p, status);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_t(const T* value, const T* om, T* out, const DcnParams& p, int* status, cudaStream_t s) {
  return p.vb == 32 ? launch_vb<T, 32>(value, om, out, p, status, s)
                    : launch_vb<T, 16>(value, om, out, p, status, s);
}

cudaError_t launch_dcnv4_fwd(int dtype, const void* value, const void* om, void* out,
                             const DcnParams& p, int* status, cudaStream_t s) {
  switch (dtype) {
    case 0: return launch_t((const float*)value, (const float*)om, (float*)out, p, status, s);
    case 1: return launch_t((const __half*)value, (const __half*)om, (__half*)out, p, status, s);
    default: return launch_t((const __nv_bfloat16*)value, (const __nv_bfloat16*)om, (__nv_bfloat16*)out, p, status, s);
  }
}

}  // namespace dcnb200
