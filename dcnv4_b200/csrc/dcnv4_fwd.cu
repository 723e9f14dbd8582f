// DCNv4 forward: out[b,y,x,g,:] = sum_k mask_k * bilinear(value[b,:,:,g,:], h_k, w_k).
//
// Replaces the reference's forward_kernel_dcn_reg + launcher
// (DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:142-325) and the zero-filled output of its host
// wrapper (DCNv4_op/src/cuda/dcnv4_cuda.cu:62): every output element is written exactly
// once, so no memset is needed.
//
// Work decomposition: a CTA takes `tile` consecutive queries (flat index over N*Ho*Wo, so a
// tile may cross rows and images freely -- batch and position are derived per query from
// the flat index).  Their packed offset/mask rows are one contiguous span staged to shared
// memory by a single bulk copy.  Work items (query, group, channel vector) are laid out
// channel-fastest so a warp's output store covers consecutive bytes.
#include "common.cuh"

namespace dcnb200 {

size_t dcnv4_fwd_smem(const DcnParams& p, int elem) {
  size_t b = 16 + (size_t)p.tile * p.Ppad * elem;
  if (p.softmax) b += (size_t)p.tile * p.G * sizeof(float2);
  return b;
}

template <typename T, int KH, int KW>
__global__ void __launch_bounds__(kThreads)
dcnv4_fwd_kernel(const T* __restrict__ value, const T* __restrict__ om, T* __restrict__ out,
                 const DcnParams p, int* status) {
  constexpr int V = Vec<T>::N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw);
  T* s_om = reinterpret_cast<T*>(smem_raw + 16);
  float2* s_stat = reinterpret_cast<float2*>(smem_raw + 16 + (size_t)p.tile * p.Ppad * sizeof(T));

  const int q0 = blockIdx.x * p.tile;
  const int nq_tile = min(p.tile, p.nq - q0);
  if (!stage_span(s_om, om + (size_t)q0 * p.Ppad, (uint32_t)(nq_tile * p.Ppad * sizeof(T)), bar, status)) return;

  const int kh = KH ? KH : p.kh, kw = KW ? KW : p.kw;
  const int K = p.K;

  if (p.softmax) {  // per pair: max and 1/sum(exp) of the K mask logits
    for (int pr = threadIdx.x; pr < nq_tile * p.G; pr += kThreads) {
      const T* row = s_om + (pr / p.G) * p.Ppad + (pr % p.G) * 3 * K + 2 * K;
      float mx = -INFINITY;
      for (int k = 0; k < K; ++k) mx = fmaxf(mx, to_f32(row[k]));
      float sum = 0.f;
      for (int k = 0; k < K; ++k) sum += __expf(to_f32(row[k]) - mx);
      s_stat[pr] = make_float2(mx, 1.f / sum);
    }
    __syncthreads();
  }

  const int cw = (p.dw * (kw - 1)) >> 1, ch = (p.dh * (kh - 1)) >> 1;
  const int center = (kw / 2) * kh + (kh / 2);
  const int QW = p.Ho * p.Wo;
  const int n_items = nq_tile * p.G * p.tpg;

  for (int item = threadIdx.x; item < n_items; item += kThreads) {
    const int c = item % p.tpg;
    const int pr = item / p.tpg;
    const int g = pr % p.G;
    const int ql = pr / p.G;
    const int q = q0 + ql;
    const int b = q / QW;
    const int rem = q - b * QW;
    const int y = rem / p.Wo;
    const int x = rem - y * p.Wo;

    const T* row = s_om + ql * p.Ppad + g * 3 * K;
    const float base_w = dcn_base(cw - p.pw + x * p.sw, cw, p.scale);
    const float base_h = dcn_base(ch - p.ph + y * p.sh, ch, p.scale);
    float2 stat = make_float2(0.f, 1.f);
    if (p.softmax) stat = s_stat[pr];

    for (int ci = 0; ci < p.chunks; ++ci) {
      const int ch0 = (c + ci * p.tpg) * V;
      const T* img = value + (size_t)b * p.H * p.W * p.C + g * p.D + ch0;
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
          const float w_im = dcn_coord(base_w, i * p.dw, to_f32(row[2 * k]), p.scale);
          const float h_im = dcn_coord(base_h, j * p.dh, to_f32(row[2 * k + 1]), p.scale);
          float m = to_f32(row[2 * K + k]);
          if (p.softmax) m = __expf(m - stat.x) * stat.y;
          const bool ok = in_range(h_im, w_im, p.H, p.W);
          const Footprint f = footprint(h_im, w_im, p.H, p.W);
          const T* p1 = img + ((ptrdiff_t)f.h0 * p.W + f.w0) * p.C;
          const uint4 r1 = ldg_vec(p1, ok && f.top && f.left);
          const uint4 r2 = ldg_vec(p1 + p.C, ok && f.top && f.right);
          const uint4 r3 = ldg_vec(p1 + (size_t)p.W * p.C, ok && f.bot && f.left);
          const uint4 r4 = ldg_vec(p1 + (size_t)p.W * p.C + p.C, ok && f.bot && f.right);
          const float w1 = m * f.hh * f.hw, w2 = m * f.hh * f.lw, w3 = m * f.lh * f.hw, w4 = m * f.lh * f.lw;
          float v1[V], v2[V], v3[V], v4[V];
          unpack(r1, v1, (const T*)nullptr);
          unpack(r2, v2, (const T*)nullptr);
          unpack(r3, v3, (const T*)nullptr);
          unpack(r4, v4, (const T*)nullptr);
#pragma unroll
          for (int e = 0; e < V; ++e)
            acc[e] = fmaf(w1, v1[e], fmaf(w2, v2[e], fmaf(w3, v3[e], fmaf(w4, v4[e], acc[e]))));
        }
      }
      *reinterpret_cast<uint4*>(out + (size_t)q * p.C + g * p.D + ch0) = pack(acc, (const T*)nullptr);
    }
  }
}

template <typename T>
static cudaError_t launch_t(const T* value, const T* om, T* out, const DcnParams& p, int* status, cudaStream_t s) {
  const int grid = (p.nq + p.tile - 1) / p.tile;
  const size_t smem = dcnv4_fwd_smem(p, sizeof(T));
  if (p.kh == 3 && p.kw == 3)
    dcnv4_fwd_kernel<T, 3, 3><<<grid, kThreads, smem, s>>>(value, om, out, p, status);
  else
    dcnv4_fwd_kernel<T, 0, 0><<<grid, kThreads, smem, s>>>(value, om, out, p, status);
  return cudaGetLastError();
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
