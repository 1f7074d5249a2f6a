// Source of cvt_rs_hw_samples.npz: sweeps cvt.rs.satfinite.e2m1x4.f32 on a B200 over structured
// and random (value, random word) pairs and dumps {n, float4 x[n], uint32 rbits[n], uint16 out[n]}.
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O2 -o probe cvt_rs_probe.cu ; run: ./probe out.bin
// The fixture keeps the two order probes, 6000 structured and 6000 random entries of that dump.
#include <cstdio>
#include <cstdint>
#include <vector>
#include <random>
#include <cuda_runtime.h>
__global__ void k(const float4* xs, const uint32_t* rb, uint16_t* out, int n){
  int i = blockIdx.x*blockDim.x+threadIdx.x; if(i>=n) return;
  float4 v = xs[i]; uint16_t r;
  asm("cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5;" : "=h"(r) : "f"(v.x),"f"(v.y),"f"(v.z),"f"(v.w),"r"(rb[i]));
  out[i]=r;
}
int main(int argc,char**argv){
  std::vector<float4> xs; std::vector<uint32_t> rb;
  const float lv[8]={0,.5f,1,1.5f,2,3,4,6};
  // A: order
  xs.push_back({0.5f,1.0f,2.0f,4.0f}); rb.push_back(0);
  xs.push_back({-0.5f,1.5f,-3.0f,6.0f}); rb.push_back(0);
  // B: structured
  std::vector<uint32_t> pats; pats.push_back(0); pats.push_back(0xFFFFFFFFu);
  for(int b=0;b<32;b++){ pats.push_back(1u<<b); pats.push_back(~(1u<<b)); pats.push_back((1u<<b)-1u);}
  for(int p=0;p<4;p++) for(int iv=0;iv<7;iv++) for(int kf=0;kf<256;kf++){
    float x = lv[iv] + (lv[iv+1]-lv[iv])*(kf/256.0f);
    for(uint32_t pat: pats){ float4 v={0.f,0.f,0.f,0.f}; ((float*)&v)[p]=x; xs.push_back(v); rb.push_back(pat);} }
  // B2: fine fractions near 0 and 1 of interval [1,1.5] and [4,6], position 0..3, field sweeps of each byte
  for(int p=0;p<4;p++) for(int iv: {2,6}) for(int e=1;e<=22;e++){
    float x = lv[iv] + (lv[iv+1]-lv[iv])*ldexpf(1.f,-e);
    float x2 = lv[iv+1] - (lv[iv+1]-lv[iv])*ldexpf(1.f,-e);
    for(uint32_t pat: pats){ float4 v={0,0,0,0}; ((float*)&v)[p]=x; xs.push_back(v); rb.push_back(pat);
                             float4 w={0,0,0,0}; ((float*)&w)[p]=x2; xs.push_back(w); rb.push_back(pat);} }
  size_t nstruct = xs.size();
  // C: random
  std::mt19937 g(123); std::uniform_real_distribution<float> U(-7.f,7.f);
  for(int i=0;i<400000;i++){ xs.push_back({U(g),U(g),U(g),U(g)}); rb.push_back(g()); }
  int n = xs.size();
  float4* dx; uint32_t* dr; uint16_t* dout;
  cudaMalloc(&dx,n*sizeof(float4)); cudaMalloc(&dr,n*4); cudaMalloc(&dout,n*2);
  cudaMemcpy(dx,xs.data(),n*sizeof(float4),cudaMemcpyHostToDevice); cudaMemcpy(dr,rb.data(),n*4,cudaMemcpyHostToDevice);
  k<<<(n+255)/256,256>>>(dx,dr,dout,n);
  std::vector<uint16_t> out(n); cudaError_t e=cudaMemcpy(out.data(),dout,n*2,cudaMemcpyDeviceToHost);
  printf("n=%d nstruct=%zu err=%s\n",n,nstruct,cudaGetErrorString(e));
  printf("order: in (0.5,1,2,4) -> 0x%04x ; (-0.5,1.5,-3,6) -> 0x%04x\n", out[0], out[1]);
  FILE* f=fopen(argc>1?argv[1]:"cvt_probe.bin","wb");
  fwrite(&n,4,1,f); fwrite(xs.data(),sizeof(float4),n,f); fwrite(rb.data(),4,n,f); fwrite(out.data(),2,n,f); fclose(f);
  return 0;
}
