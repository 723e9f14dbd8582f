// DCNv4 backward: grad_value (scatter) and grad_offset_mask (per-point reductions).
//
// Replaces backward_kernel_dcn_warp_primitive / backward_kernel_dcn and their launcher
// (DCNv4_op/src/cuda/dcnv4_col2im_cuda.cuh:20-472, helper DCNv4_op/src/cuda/common.h:100-212)
// plus the zero-fills and the fp16 cast passes of the host wrapper
// (DCNv4_op/src/cuda/dcnv4_cuda.cu:133-139,169-174).
//
//  * grad_value contributions go to an fp32 accumulation buffer with 16-byte vector
//    reductions (red.global.add.v4.f32), one per corner and channel vector, instead of one
//    scalar atomic per element.
//  * The three per-point partials (d/dx, d/dy, d/dmask) are reduced over the lanes of a pair
//    with warp shuffles.  Lane 0 of the pair deposits them in a shared-memory image of the
//    tile's grad_offset_mask rows; the CTA then writes whole rows (pad columns included, as
//    zeros) with coalesced 16-byte stores, so grad_offset_mask needs no memset either.
#include "common.cuh"

namespace dcnb200 {

size_t dcnv4_bwd_smem(const DcnParams& p, int elem) {
  size_t b = 16 + (size_t)p.tile * p.Ppad * elem + (size_t)p.tile * p.Ppad * sizeof(float);
  if (p.softmax) b += (size_t)p.tile * p.G * sizeof(float2);
  return b;
}

template <typename T, int KH, int KW, bool ONE_CHUNK>
__global__ void __launch_bounds__(kThreads)
dcnv4_bwd_kernel(const T* __restrict__ value, const T* __restrict__ om, const T* __restrict__ gout,
                 float* __restrict__ gvalue, T* __restrict__ gom, const DcnParams p, int* status) {
  constexpr int V = Vec<T>::N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw);
  T* s_om = reinterpret_cast<T*>(smem_raw + 16);
  float* s_g = reinterpret_cast<float*>(smem_raw + 16 + (size_t)p.tile * p.Ppad * sizeof(T));
  float2* s_stat = reinterpret_cast<float2*>(s_g + (size_t)p.tile * p.Ppad);

  const int q0 = blockIdx.x * p.tile;
  const int nq_tile = min(p.tile, p.nq - q0);
  if (!stage_span(s_om, om + (size_t)q0 * p.Ppad, (uint32_t)(nq_tile * p.Ppad * sizeof(T)), bar, status)) return;

  const int kh = KH ? KH : p.kh, kw = KW ? KW : p.kw;
  const int K = p.K;
  const int used = 3 * K * p.G;

  // pad columns of the gradient rows are zeros
  for (int i = threadIdx.x; i < nq_tile * (p.Ppad - used); i += kThreads)
    s_g[(i / (p.Ppad - used)) * p.Ppad + used + i % (p.Ppad - used)] = 0.f;

  if (p.softmax) {
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

  // Every lane of a warp takes part in the shuffles, so the loop runs over whole CTA-wide
  // strides and lanes past the end work on item 0 with all memory traffic disabled.
  for (int base = 0; base < n_items; base += kThreads) {
    const bool active = base + threadIdx.x < n_items;
    const int item = active ? base + threadIdx.x : 0;
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
    float* grow = s_g + ql * p.Ppad + g * 3 * K;
    const float base_w = dcn_base(cw - p.pw + x * p.sw, cw, p.scale);
    const float base_h = dcn_base(ch - p.ph + y * p.sh, ch, p.scale);
    float2 stat = make_float2(0.f, 1.f);
    if (p.softmax) stat = s_stat[pr];

    const size_t img_off = (size_t)b * p.H * p.W * p.C + g * p.D;
    const T* go_ptr = gout + (size_t)q * p.C + g * p.D;
    float gy0[V];
    if (ONE_CHUNK) unpack(ldg_vec(go_ptr + c * V, active), gy0, (const T*)nullptr);

    float soft_sum = 0.f;  // sum_k t_k (softmax backward), kept by lane 0 of the pair
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
        const bool ok = active && in_range(h_im, w_im, p.H, p.W);
        const Footprint f = footprint(h_im, w_im, p.H, p.W);
        const ptrdiff_t pix = ((ptrdiff_t)f.h0 * p.W + f.w0) * p.C;
        const bool ok1 = ok && f.top && f.left, ok2 = ok && f.top && f.right;
        const bool ok3 = ok && f.bot && f.left, ok4 = ok && f.bot && f.right;
        const float w1 = f.hh * f.hw, w2 = f.hh * f.lw, w3 = f.lh * f.hw, w4 = f.lh * f.lw;

        float d1 = 0.f, d2 = 0.f, d3 = 0.f, d4 = 0.f;  // sum_c gy_c * v_corner,c
        const int n_chunks = ONE_CHUNK ? 1 : p.chunks;
        for (int ci = 0; ci < n_chunks; ++ci) {
          const int ch0 = (c + ci * p.tpg) * V;
          float gy[V];
          if (ONE_CHUNK) {
#pragma unroll
            for (int e = 0; e < V; ++e) gy[e] = gy0[e];
          } else {
            unpack(ldg_vec(go_ptr + ch0, active), gy, (const T*)nullptr);
          }
          const T* p1 = value + img_off + ch0 + pix;
          const uint4 r1 = ldg_vec(p1, ok1);
          const uint4 r2 = ldg_vec(p1 + p.C, ok2);
          const uint4 r3 = ldg_vec(p1 + (size_t)p.W * p.C, ok3);
          const uint4 r4 = ldg_vec(p1 + (size_t)p.W * p.C + p.C, ok4);
          float* a1 = gvalue + img_off + ch0 + pix;
          const float s1 = m * w1, s2 = m * w2, s3 = m * w3, s4 = m * w4;
#pragma unroll
          for (int e = 0; e < V; e += 4) {
            if (ok1) red_add_v4(a1 + e, s1 * gy[e], s1 * gy[e + 1], s1 * gy[e + 2], s1 * gy[e + 3]);
            if (ok2) red_add_v4(a1 + p.C + e, s2 * gy[e], s2 * gy[e + 1], s2 * gy[e + 2], s2 * gy[e + 3]);
            if (ok3) red_add_v4(a1 + (size_t)p.W * p.C + e, s3 * gy[e], s3 * gy[e + 1], s3 * gy[e + 2], s3 * gy[e + 3]);
            if (ok4) red_add_v4(a1 + (size_t)p.W * p.C + p.C + e, s4 * gy[e], s4 * gy[e + 1], s4 * gy[e + 2], s4 * gy[e + 3]);
          }
          float v1[V], v2[V], v3[V], v4[V];
          unpack(r1, v1, (const T*)nullptr);
          unpack(r2, v2, (const T*)nullptr);
          unpack(r3, v3, (const T*)nullptr);
          unpack(r4, v4, (const T*)nullptr);
#pragma unroll
          for (int e = 0; e < V; ++e) {
            d1 = fmaf(gy[e], v1[e], d1);
            d2 = fmaf(gy[e], v2[e], d2);
            d3 = fmaf(gy[e], v3[e], d3);
            d4 = fmaf(gy[e], v4[e], d4);
          }
        }
        // d/dw, d/dh of the bilinear value and the value itself, dotted with gy
        float gx = f.hh * (d2 - d1) + f.lh * (d4 - d3);
        float gyv = f.hw * (d3 - d1) + f.lw * (d4 - d2);
        float gm = w1 * d1 + w2 * d2 + w3 * d3 + w4 * d4;
        for (int o = p.tpg >> 1; o > 0; o >>= 1) {
          gx += __shfl_xor_sync(0xffffffffu, gx, o);
          gyv += __shfl_xor_sync(0xffffffffu, gyv, o);
          gm += __shfl_xor_sync(0xffffffffu, gm, o);
        }
        if (active && c == 0) {
          grow[2 * k] = ok ? p.scale * m * gx : 0.f;
          grow[2 * k + 1] = ok ? p.scale * m * gyv : 0.f;
          const float gmk = ok ? gm : 0.f;
          if (p.softmax) {
            grow[2 * K + k] = gmk * m;
            soft_sum += gmk * m;
          } else {
            grow[2 * K + k] = gmk;
          }
        }
      }
    }
    if (p.softmax && active && c == 0) {
      for (int k = 0; k < K; ++k) {
        const float m = __expf(to_f32(row[2 * K + k]) - stat.x) * stat.y;
        grow[2 * K + k] -= m * soft_sum;
      }
    }
  }

  __syncthreads();
  // coalesced write-out of the tile's grad_offset_mask rows
  const int n_vec = nq_tile * p.Ppad / V;
  T* dst = gom + (size_t)q0 * p.Ppad;
  for (int i = threadIdx.x; i < n_vec; i += kThreads) {
    float v[V];
#pragma unroll
    for (int e = 0; e < V; e += 4) {
      const float4 f4 = *reinterpret_cast<const float4*>(s_g + (size_t)i * V + e);
      v[e] = f4.x; v[e + 1] = f4.y; v[e + 2] = f4.z; v[e + 3] = f4.w;
    }
    *reinterpret_cast<uint4*>(dst + (size_t)i * V) = pack(v, (const T*)nullptr);
  }
}

template <typename T>
static cudaError_t launch_t(const T* value, const T* om, const T* gout, float* gvalue, T* gom,
                            const DcnParams& p, int* status, cudaStream_t s) {
  const int grid = (p.nq + p.tile - 1) / p.tile;
  const size_t smem = dcnv4_bwd_smem(p, sizeof(T));
  const bool k33 = p.kh == 3 && p.kw == 3;
  if (k33 && p.chunks == 1)
    dcnv4_bwd_kernel<T, 3, 3, true><<<grid, kThreads, smem, s>>>(value, om, gout, gvalue, gom, p, status);
  else if (k33)
    dcnv4_bwd_kernel<T, 3, 3, false><<<grid, kThreads, smem, s>>>(value, om, gout, gvalue, gom, p, status);
  else
    dcnv4_bwd_kernel<T, 0, 0, false><<<grid, kThreads, smem, s>>>(value, om, gout, gvalue, gom, p, status);
  return cudaGetLastError();
}

cudaError_t launch_dcnv4_bwd(int dtype, const void* value, const void* om, const void* gout,
                             float* gvalue_f32, void* gom, const DcnParams& p, int* status, cudaStream_t s) {
  switch (dtype) {
    case 0: return launch_t((const float*)value, (const float*)om, (const float*)gout, gvalue_f32, (float*)gom, p, status, s);
    case 1: return launch_t((const __half*)value, (const __half*)om, (const __half*)gout, gvalue_f32, (__half*)gom, p, status, s);
    default: return launch_t((const __nv_bfloat16*)value, (const __nv_bfloat16*)om, (const __nv_bfloat16*)gout, gvalue_f32, (__nv_bfloat16*)gom, p, status, s);
  }
}

}  // namespace dcnb200
