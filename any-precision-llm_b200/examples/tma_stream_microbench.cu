// Microbenchmark: how fast can bitplane operands be streamed from HBM into shared memory with tiled TMA boxes of a
// given shape and ring depth (one warp per block waits and re-arms, nothing is computed), and with plain loads?
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I include -o tma_stream_microbench any-precision-llm_b200/examples/tma_stream_microbench.cu
//   ./tma_stream_microbench N K w_bits          e.g.  ./tma_stream_microbench 4096 32768 3
// Launches are plain (no programmatic dependent launch): about 2.8 us per launch is launch overhead.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <stdint.h>
#include "../csrc/ap_tensormap.h"
#define CK(x) do{cudaError_t e=(x); if(e!=cudaSuccess){printf("err %s line %d\n",cudaGetErrorString(e),__LINE__);exit(1);}}while(0)
__device__ unsigned int sink;
__device__ __forceinline__ bool wait_b(uint32_t bar,uint32_t parity){ for(uint32_t i=0;i<(1u<<20);i++){uint32_t ok; asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}":"=r"(ok):"r"(bar),"r"(parity):"memory"); if(ok) return true;} return false; }
// A: TMA boxes [W][R rows][CW words]; one warp per CTA consumes; ring depth D
template<int D>
__global__ void __launch_bounds__(32) tma_stream(const __grid_constant__ CUtensorMap map, int W, int R, int CW, int words, int touch){
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ uint64_t bars[D];
  const int box = W*R*CW*4; const int nch = words/CW; const int row0=blockIdx.x*R;
  uint32_t sm=(uint32_t)__cvta_generic_to_shared(smem), bs=(uint32_t)__cvta_generic_to_shared(bars);
  if(threadIdx.x==0){ for(int b=0;b<D;b++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;"::"r"(bs+8*b)); asm volatile("fence.mbarrier_init.release.cluster;":::"memory");
    for(int i=0;i<D&&i<nch;i++){ asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"::"r"(bs+8*i),"r"((uint32_t)box):"memory");
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"::"r"(sm+i*box),"l"((uint64_t)&map),"r"(i*CW),"r"(row0),"r"(0),"r"(bs+8*i):"memory"); } }
  __syncwarp();
  unsigned acc=0;
  for(int i=0;i<nch;i++){ int b=i%D; if(!wait_b(bs+8*b,(i/D)&1)) break;
    if(touch){ acc += *reinterpret_cast<volatile unsigned*>(smem+b*box+threadIdx.x*4); }
    __syncwarp();
    if(threadIdx.x==0 && i+D<nch){ asm volatile("fence.proxy.async.shared::cta;":::"memory"); asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"::"r"(bs+8*b),"r"((uint32_t)box):"memory");
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"::"r"(sm+b*box),"l"((uint64_t)&map),"r"((i+D)*CW),"r"(row0),"r"(0),"r"(bs+8*b):"memory"); }
  }
  if(acc==0x12345678) sink=acc;
}
// A2: as A, but boxes are re-armed in groups of G adjacent chunks (all G consumed, then all G requested together)
template<int D,int G>
__global__ void __launch_bounds__(32) tma_stream_g(const __grid_constant__ CUtensorMap map, int W, int R, int CW, int words, int touch){
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ uint64_t bars[D];
  const int box = W*R*CW*4; const int nch = words/CW; const int row0=blockIdx.x*R;
  uint32_t sm=(uint32_t)__cvta_generic_to_shared(smem), bs=(uint32_t)__cvta_generic_to_shared(bars);
  auto req=[&](int i){ int b=i%D; asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"::"r"(bs+8*b),"r"((uint32_t)box):"memory");
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"::"r"(sm+b*box),"l"((uint64_t)&map),"r"(i*CW),"r"(row0),"r"(0),"r"(bs+8*b):"memory"); };
  if(threadIdx.x==0){ for(int b=0;b<D;b++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;"::"r"(bs+8*b)); asm volatile("fence.mbarrier_init.release.cluster;":::"memory");
    for(int i=0;i<D&&i<nch;i++) req(i); }
  __syncwarp();
  unsigned acc=0;
  for(int i0=0;i0<nch;i0+=G){
    for(int i=i0;i<i0+G&&i<nch;i++){ int b=i%D; if(!wait_b(bs+8*b,(i/D)&1)) return; if(touch) acc += *reinterpret_cast<volatile unsigned*>(smem+b*box+threadIdx.x*4); }
    __syncwarp();
    if(threadIdx.x==0){ asm volatile("fence.proxy.async.shared::cta;":::"memory"); for(int i=i0;i<i0+G;i++) if(i+D<nch) req(i+D); }
  }
  if(acc==0x12345678) sink=acc;
}
// C: plain 16-byte loads, same column-slice pattern: CTA = R rows, chunk = CW words of every row and plane; U chunks in flight per thread
template<int U>
__global__ void __launch_bounds__(256) ldg_stream(const uint4* __restrict__ q, long long plane_vecs, int W, int R, int words, int rowmajor){
  const int vecs=words/4; const int row0=blockIdx.x*R; unsigned acc=0;
  // items per chunk: W*R*8 (8 x 16B per 128B piece)
  const int items=W*R*8; const int nch=words/32;
  if(!rowmajor){
    for(int c0=0;c0<nch;c0+=U){
      uint4 v[U];
      #pragma unroll
      for(int u=0;u<U;u++){ int c=c0+u; for(int it=threadIdx.x; it<items; it+=256){ int p=it/(R*8), r=(it/8)%R, piece=it%8; if(c<nch){ uint4 t=__ldcs(q+(size_t)p*plane_vecs+(size_t)(row0+r)*vecs+c*8+piece); acc^=t.x^t.y^t.z^t.w; } } }
    }
  } else {
    // row-major: each warp walks one (plane,row) at a time, 512 B per warp-instruction
    const int warp=threadIdx.x>>5, lane=threadIdx.x&31;
    for(int pr=warp; pr<W*R; pr+=8){ int p=pr/R, r=pr%R; const uint4* src=q+(size_t)p*plane_vecs+(size_t)(row0+r)*vecs;
      for(int v0=lane; v0<vecs; v0+=32*U){
        #pragma unroll
        for(int u=0;u<U;u++){ int vi=v0+32*u; if(vi<vecs){ uint4 t=__ldcs(src+vi); acc^=t.x^t.y^t.z^t.w; } } } }
  }
  if(acc==0x12345678) sink=acc;
}
__global__ void fill(uint32_t* p,size_t n){ size_t i=blockIdx.x*(size_t)blockDim.x+threadIdx.x; size_t st=(size_t)gridDim.x*blockDim.x; for(;i<n;i+=st) p[i]=(uint32_t)i*2654435761u; }
int main(int argc,char**argv){
  int N=atoi(argv[1]),K=atoi(argv[2]),W=atoi(argv[3]); int words=K/32; const int L=6;
  uint32_t* q[L]; size_t qn=(size_t)8*N*words; for(int i=0;i<L;i++){ CK(cudaMalloc(&q[i],qn*4)); fill<<<1024,256>>>(q[i],qn);} CK(cudaDeviceSynchronize());
  cudaEvent_t e0,e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  double bytes=(double)N*K*W/8;
  ap::EncodeTiledFn enc=ap::encode_tiled_fn();
  auto run_tma=[&](int R,int CW,int D,int touch,int swz){
    CUtensorMap maps[L];
    for(int i=0;i<L;i++){ cuuint64_t dims[3]={(cuuint64_t)words,(cuuint64_t)N,(cuuint64_t)W}; cuuint64_t str[2]={(cuuint64_t)words*4,(cuuint64_t)N*words*4}; cuuint32_t box[3]={(cuuint32_t)CW,(cuuint32_t)R,(cuuint32_t)W}; cuuint32_t es[3]={1,1,1};
      CUresult r=enc(&maps[i],CU_TENSOR_MAP_DATA_TYPE_INT32,3,q[i],dims,str,box,es,CU_TENSOR_MAP_INTERLEAVE_NONE,swz?CU_TENSOR_MAP_SWIZZLE_128B:CU_TENSOR_MAP_SWIZZLE_NONE,CU_TENSOR_MAP_L2_PROMOTION_L2_256B,CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE); if(r!=CUDA_SUCCESS){printf("encode fail %d\n",(int)r);return;} }
    int box=W*R*CW*4; int smem=box*D+1024;
    auto launch=[&](int i){ switch(D){
      case 2: cudaFuncSetAttribute(tma_stream<2>,cudaFuncAttributeMaxDynamicSharedMemorySize,smem); tma_stream<2><<<N/R,32,smem>>>(maps[i],W,R,CW,words,touch); break;
      case 4: cudaFuncSetAttribute(tma_stream<4>,cudaFuncAttributeMaxDynamicSharedMemorySize,smem); tma_stream<4><<<N/R,32,smem>>>(maps[i],W,R,CW,words,touch); break;
      case 8: cudaFuncSetAttribute(tma_stream<8>,cudaFuncAttributeMaxDynamicSharedMemorySize,smem); tma_stream<8><<<N/R,32,smem>>>(maps[i],W,R,CW,words,touch); break;
      case 16: cudaFuncSetAttribute(tma_stream<16>,cudaFuncAttributeMaxDynamicSharedMemorySize,smem); tma_stream<16><<<N/R,32,smem>>>(maps[i],W,R,CW,words,touch); break; } };
    if(smem>220*1024){printf("tma R=%d CW=%d D=%d: too much smem\n",R,CW,D);return;}
    for(int i=0;i<L;i++) launch(i); CK(cudaDeviceSynchronize());
    cudaEventRecord(e0); for(int it=0;it<3;it++) for(int i=0;i<L;i++) launch(i); cudaEventRecord(e1); CK(cudaDeviceSynchronize());
    float ms; cudaEventElapsedTime(&ms,e0,e1); double us=ms*1e3/(3*L);
    printf("tma  R=%3d CW=%3d D=%2d touch=%d swz=%d smem=%6d: %7.2f us  %6.0f GB/s\n",R,CW,D,touch,swz,smem,us,bytes/us/1e3);
  };
  auto run_tmag=[&](int R,int CW,int promo){
    constexpr int D=8,G=4;
    CUtensorMap maps[L];
    for(int i=0;i<L;i++){ cuuint64_t dims[3]={(cuuint64_t)words,(cuuint64_t)N,(cuuint64_t)W}; cuuint64_t str[2]={(cuuint64_t)words*4,(cuuint64_t)N*words*4}; cuuint32_t box[3]={(cuuint32_t)CW,(cuuint32_t)R,(cuuint32_t)W}; cuuint32_t es[3]={1,1,1};
      CUresult r=enc(&maps[i],CU_TENSOR_MAP_DATA_TYPE_INT32,3,q[i],dims,str,box,es,CU_TENSOR_MAP_INTERLEAVE_NONE,CU_TENSOR_MAP_SWIZZLE_128B,promo==0?CU_TENSOR_MAP_L2_PROMOTION_NONE:promo==1?CU_TENSOR_MAP_L2_PROMOTION_L2_128B:CU_TENSOR_MAP_L2_PROMOTION_L2_256B,CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE); if(r!=CUDA_SUCCESS){printf("encode fail %d\n",(int)r);return;} }
    int box=W*R*CW*4; int smem=box*D+1024; if(smem>220*1024){printf("tmag too much smem\n");return;}
    cudaFuncSetAttribute(tma_stream_g<D,G>,cudaFuncAttributeMaxDynamicSharedMemorySize,smem);
    auto launch=[&](int i){ tma_stream_g<D,G><<<N/R,32,smem>>>(maps[i],W,R,CW,words,1); };
    for(int i=0;i<L;i++) launch(i); CK(cudaDeviceSynchronize());
    cudaEventRecord(e0); for(int it=0;it<3;it++) for(int i=0;i<L;i++) launch(i); cudaEventRecord(e1); CK(cudaDeviceSynchronize());
    float ms; cudaEventElapsedTime(&ms,e0,e1); double us=ms*1e3/(3*L);
    printf("tmaG R=%3d CW=%3d D=8 G=4 promo=%d: %7.2f us  %6.0f GB/s\n",R,CW,promo,us,bytes/us/1e3);
  };
  auto run_ldg=[&](int R,int U,int rowmajor){
    auto launch=[&](int i){ if(U==1) ldg_stream<1><<<N/R,256>>>((const uint4*)q[i],(long long)N*words/4,W,R,words,rowmajor); else if(U==2) ldg_stream<2><<<N/R,256>>>((const uint4*)q[i],(long long)N*words/4,W,R,words,rowmajor); else ldg_stream<4><<<N/R,256>>>((const uint4*)q[i],(long long)N*words/4,W,R,words,rowmajor); };
    for(int i=0;i<L;i++) launch(i); CK(cudaDeviceSynchronize());
    cudaEventRecord(e0); for(int it=0;it<3;it++) for(int i=0;i<L;i++) launch(i); cudaEventRecord(e1); CK(cudaDeviceSynchronize());
    float ms; cudaEventElapsedTime(&ms,e0,e1); double us=ms*1e3/(3*L);
    printf("ldg  R=%3d U=%d rowmajor=%d: %7.2f us  %6.0f GB/s\n",R,U,rowmajor,us,bytes/us/1e3);
  };
  printf("N=%d K=%d W=%d  bytes=%.1f MB\n",N,K,W,bytes/1e6);
  run_tmag(16,32,2); run_tmag(16,32,1); run_tmag(16,32,0);
  for(int D: {2,4,8,16}) run_tma(16,32,D,1,1);
  run_tma(16,32,8,0,1);
  run_tma(16,32,8,1,0);
  for(int D: {2,4,8}) run_tma(32,32,D,1,1);
  for(int D: {2,4}) run_tma(64,32,D,1,1);
  run_tma(16,64,4,1,0); run_tma(16,128,4,1,0); run_tma(16,256,2,1,0);
  run_tma(8,32,8,1,1); run_tma(8,32,16,1,1);
  for(int U: {1,2,4}) run_ldg(16,U,0);
  for(int U: {1,2,4}) run_ldg(16,U,1);
  return 0;
}
