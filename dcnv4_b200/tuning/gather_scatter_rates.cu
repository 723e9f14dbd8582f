// Stand-alone rate measurements behind the lane geometry of the DCNv4 / FlashDeformAttn kernels.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o gather_scatter_rates gather_scatter_rates.cu
//   ./gather_scatter_rates
//
// Every test moves random 64-byte "groups" (16 fp32 channels of one pixel of one group -- what a
// bilinear corner of a (query, group) pair is at D=16) between registers and a 512-pixel window,
// from 4 CTAs of 256 threads per SM, and prints groups per second and per SM-cycle:
//   * read-only global gathers (L1-resident window) with 4, 2 or 1 lanes per group,
//   * shared-memory gathers,
//   * vector reductions to global memory (red.global.add.v4.f32, 4 lanes per group),
//   * shared-memory reductions: float (compare-and-swap loop), 32-bit integer, plain
//     read-modify-write.
// Results on B200 are summarised in profiles/b200_gather_scatter_rates.md.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do{cudaError_t e=(x); if(e!=cudaSuccess){printf("err %s line %d\n",cudaGetErrorString(e),__LINE__); return 1;}}while(0)
__device__ __forceinline__ uint32_t rng(uint32_t& s){ s = s*1664525u+1013904223u; return s>>8; }

// each thread: iters x 16 scalar float atomicAdds to smem at random pixel (64B groups), 4 lanes per pixel
__global__ void k_smem_atomic(float* out, int iters, int npix){
  extern __shared__ float sm[];
  for(int i=threadIdx.x;i<npix*16;i+=blockDim.x) sm[i]=0.f;
  __syncthreads();
  uint32_t s = (blockIdx.x*blockDim.x+threadIdx.x)/4*7919u+1;  // same seed for 4 lanes of a "pair"
  int c = threadIdx.x&3;
  for(int it=0;it<iters;++it){
    int pix = rng(s)%npix;
    float* p = sm + pix*16 + c*4;
    atomicAdd(p+0, 1.f); atomicAdd(p+1, 1.f); atomicAdd(p+2, 1.f); atomicAdd(p+3, 1.f);
  }
  __syncthreads();
  if(threadIdx.x==0) out[blockIdx.x]=sm[0];
}
// global red.v4: 4 lanes per 64B group at random pixel within a window (npix groups per block region)
__global__ void k_gred(float* buf, int iters, int npix_total){
  uint32_t s = (blockIdx.x*blockDim.x+threadIdx.x)/4*7919u+1;
  int c = threadIdx.x&3;
  for(int it=0;it<iters;++it){
    int pix = rng(s)%npix_total;
    float* p = buf + (size_t)pix*16 + c*4;
    asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};"::"l"(p),"f"(1.f),"f"(1.f),"f"(1.f),"f"(1.f):"memory");
  }
}
// LDG gather: LANES lanes per 64B group, random pixel in a window of npix (fits L1)
template<int LANES>
__global__ void k_ldg(const float* buf, float* out, int iters, int npix){
  uint32_t s = (blockIdx.x*blockDim.x+threadIdx.x)/LANES*7919u+1;
  int c = threadIdx.x%LANES;
  const float* base = buf + (size_t)(blockIdx.x%148)*npix*16;
  float acc=0;
  for(int it=0;it<iters;++it){
    int pix = rng(s)%npix;
    if(LANES==4){ float4 v = __ldg((const float4*)(base + pix*16 + c*4)); acc += v.x+v.y+v.z+v.w; }
    else if(LANES==2){ float4 v = __ldg((const float4*)(base + pix*16 + c*8)); float4 w=__ldg((const float4*)(base + pix*16 + c*8+4)); acc += v.x+v.y+v.z+v.w+w.x+w.w; }
    else { for(int q=0;q<4;++q){ float4 v = __ldg((const float4*)(base + pix*16 + q*4)); acc += v.x+v.w; } }
  }
  out[blockIdx.x*blockDim.x+threadIdx.x]=acc;
}
// LDS gather: 4 lanes per 64B group from smem tile
__global__ void k_lds(const float* buf, float* out, int iters, int npix){
  extern __shared__ float sm[];
  for(int i=threadIdx.x;i<npix*16;i+=blockDim.x) sm[i]=buf[i];
  __syncthreads();
  uint32_t s = (blockIdx.x*blockDim.x+threadIdx.x)/4*7919u+1;
  int c = threadIdx.x&3;
  float acc=0;
  for(int it=0;it<iters;++it){
    int pix = rng(s)%npix;
    float4 v = *(const float4*)(sm + pix*16 + c*4); acc += v.x+v.y+v.z+v.w;
  }
  out[blockIdx.x*blockDim.x+threadIdx.x]=acc;
}
// MODE 0: int atomicAdd x4 per lane; MODE 1: red.shared.add.f32 x4; MODE 2: red.shared.add.u32 via PTX; MODE 3: plain LDS.128+STS.128 RMW (non-atomic)
template<int MODE>
__global__ void k_smem_red(float* out, int iters, int npix){
  extern __shared__ float sm[];
  for(int i=threadIdx.x;i<npix*16;i+=blockDim.x) sm[i]=0.f;
  __syncthreads();
  uint32_t s = (blockIdx.x*blockDim.x+threadIdx.x)/4*7919u+1;
  int c = threadIdx.x&3;
  for(int it=0;it<iters;++it){
    int pix = rng(s)%npix;
    float* p = sm + pix*16 + c*4;
    if(MODE==0){ int* q=(int*)p; atomicAdd(q+0,1); atomicAdd(q+1,2); atomicAdd(q+2,3); atomicAdd(q+3,4); }
    else if(MODE==1){ uint32_t a=(uint32_t)__cvta_generic_to_shared(p);
      asm volatile("red.shared.add.f32 [%0], %1;"::"r"(a),"f"(1.f):"memory"); asm volatile("red.shared.add.f32 [%0], %1;"::"r"(a+4),"f"(1.f):"memory");
      asm volatile("red.shared.add.f32 [%0], %1;"::"r"(a+8),"f"(1.f):"memory"); asm volatile("red.shared.add.f32 [%0], %1;"::"r"(a+12),"f"(1.f):"memory"); }
    else if(MODE==2){ uint32_t a=(uint32_t)__cvta_generic_to_shared(p);
      asm volatile("red.shared.add.u32 [%0], %1;"::"r"(a),"r"(1):"memory"); asm volatile("red.shared.add.u32 [%0], %1;"::"r"(a+4),"r"(1):"memory");
      asm volatile("red.shared.add.u32 [%0], %1;"::"r"(a+8),"r"(1):"memory"); asm volatile("red.shared.add.u32 [%0], %1;"::"r"(a+12),"r"(1):"memory"); }
    else { float4 v=*(float4*)p; v.x+=1.f; v.y+=1.f; v.z+=1.f; v.w+=1.f; *(float4*)p=v; }
  }
  __syncthreads();
  if(threadIdx.x==0) out[blockIdx.x]=sm[0];
}
// 64-bit packed int atomics: 2 per lane (atom.shared.add.u64)
__global__ void k64(float* out, int iters, int npix){
  extern __shared__ float sm[];
  for(int i=threadIdx.x;i<npix*16;i+=blockDim.x) sm[i]=0.f;
  __syncthreads();
  uint32_t s = (blockIdx.x*blockDim.x+threadIdx.x)/4*7919u+1;
  int c = threadIdx.x&3;
  for(int it=0;it<iters;++it){
    int pix = rng(s)%npix;
    unsigned long long* p = (unsigned long long*)(sm + pix*16 + c*4);
    atomicAdd(p, 0x0000000100000001ULL); atomicAdd(p+1, 0x0000000100000001ULL);
  }
  __syncthreads();
  if(threadIdx.x==0) out[blockIdx.x]=sm[0];
}
int main(){
  float *buf,*out; CK(cudaMalloc(&buf, 256<<20)); CK(cudaMalloc(&out, 64<<20)); CK(cudaMemset(buf,0,256<<20));
  cudaEvent_t e0,e1; cudaEventCreate(&e0); cudaEventCreate(&e1); float ms;
  int blocks=148*4, threads=256, iters=2000;
  #define TIME(name, call, ops) for(int r=0;r<2;++r){ cudaEventRecord(e0); call; cudaEventRecord(e1); CK(cudaEventSynchronize(e1)); cudaEventElapsedTime(&ms,e0,e1);} printf("%-28s %8.3f ms  %8.2f G group-ops/s  (%.2f per SM-cycle @1.9GHz)\n", name, ms, (ops)/ms/1e6, (ops)/ms/1e6/148/1.9);
  double groups = (double)blocks*threads/4*iters;
  CK(cudaFuncSetAttribute(k_smem_atomic, cudaFuncAttributeMaxDynamicSharedMemorySize, 64*1024));
  TIME("smem float atomic 16ch", (k_smem_atomic<<<blocks,threads,512*64>>>(out,iters,512)), groups);
  TIME("global red.v4 (51MB target)", (k_gred<<<blocks,threads>>>(buf,iters,802816)), groups);
  TIME("global red.v4 (local 4MB)", (k_gred<<<blocks,threads>>>(buf,iters,65536)), groups);
  TIME("LDG 4 lanes x16B / 64B", (k_ldg<4><<<blocks,threads>>>(buf,out,iters,512)), groups);
  TIME("LDG 2 lanes x32B / 64B", (k_ldg<2><<<blocks,threads>>>(buf,out,iters,512)), (double)blocks*threads/2*iters);
  TIME("LDG 1 lane  x64B / 64B", (k_ldg<1><<<blocks,threads>>>(buf,out,iters,512)), (double)blocks*threads*iters);
  CK(cudaFuncSetAttribute(k_lds, cudaFuncAttributeMaxDynamicSharedMemorySize, 64*1024));
  TIME("LDS 4 lanes x16B / 64B", (k_lds<<<blocks,threads,512*64>>>(buf,out,iters,512)), groups);
  TIME("smem int atomicAdd x4/lane", (k_smem_red<0><<<blocks,threads,512*64>>>(out,iters,512)), groups);
  TIME("smem red.shared.add.f32 x4", (k_smem_red<1><<<blocks,threads,512*64>>>(out,iters,512)), groups);
  TIME("smem red.shared.add.u32 x4", (k_smem_red<2><<<blocks,threads,512*64>>>(out,iters,512)), groups);
  TIME("smem LDS128+STS128 (non-atomic)", (k_smem_red<3><<<blocks,threads,512*64>>>(out,iters,512)), groups);
  TIME("smem atom u64 x2/lane", (k64<<<blocks,threads,512*64>>>(out,iters,512)), groups);
  return 0;
}
