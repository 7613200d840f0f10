// Shared by the hyb_*.cu operators (libpie_b200_hybrid.so): status / launch bookkeeping and typed loads.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pie_b200_hybrid.h"

namespace pieh {

int status_of(cudaError_t e);   // cudaError_t -> pie_status, remembering the message
void count_launch(int n = 1);
int num_sms();
bool pdl_enabled();   // pieh_set_pdl: launch every step operator as a programmatic dependent of the one before it

// Top of every step kernel.  Launched as a programmatic dependent, a grid may become resident while the grid before it is
// still draining: it lets ITS dependents queue up at once and then waits until everything earlier in the stream has
// completed and is visible.  Every kernel of a step does this, so completion stays transitive along the stream.
// Launched the ordinary way both instructions do nothing.
__device__ __forceinline__ void pdl_sync() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// one pieh_linear call
struct LinArgs {
  void* out; long long out_ld;
  const void* x; long long x_ld;
  const void* w;
  const float* bias;
  int M, N, K, epi;
  float epi_a;
  const float* mix; const float* outw; int S;
  float epi_b = 1.f, epi_c = 0.f;           // GLU: slope inside the sigmoid, offset of the linear half (epi_a: clamp, 0 = none)
  // grouped mode (mixture of experts): the M rows are SLOTS sorted by expert
  const int32_t* g_tiles = nullptr;         // [count, (expert, first slot, slots) ...]: blockIdx.y indexes the list
  const int32_t* g_tiles128 = nullptr;      // the same runs cut into <= 128 slots (host side: which list a kernel gets)
  const int32_t* g_rows = nullptr;          // x row of each slot (NULL: the slot itself)
  const int32_t* g_expert = nullptr;        // expert of each slot (the decode kernel: one slot per blockIdx.y)
  long long g_wstride = 0;                  // elements between two experts' matrices
  // batched mode (pieh_linear_batched): blockIdx.z picks one of nb independent products
  long long x_bs = 0, w_bs = 0, out_bs = 0; // elements between two products' operands
  const float* gate = nullptr;              // SIGMUL: fp32 logits, element z * gate_bs + m * gate_ld + n
  long long gate_ld = 0, gate_bs = 0;
  int nb = 1;
};

// the gated pair of PIEH_EPI_GLU: g the gate column, u the linear one
__device__ __forceinline__ float glu_pair(const LinArgs& a, float g, float u) {
  if (a.epi_a > 0.f) { g = fminf(g, a.epi_a); u = fminf(fmaxf(u, -a.epi_a), a.epi_a); }
  return g / (1.f + expf(-a.epi_b * g)) * (u + a.epi_c);
}

template <typename T> struct elem;
template <> struct elem<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
  static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct elem<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// sum over the whole CTA (blockDim.x a multiple of 32, <= 1024); `red` holds 33 floats; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float s = l < nw ? red[l] : 0.f;
    s = warp_sum(s);
    if (l == 0) red[32] = s;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
// a z^2 + z / 2 above zero, b (e^z - 1 - z) + z / 2 at and below it (continuous, slope 1/2 at zero from both sides)
__device__ __forceinline__ float xielu_f(float z, float a, float b) {
  return z > 0.f ? fmaf(a * z, z, 0.5f * z) : fmaf(b, expm1f(z) - z, 0.5f * z);
}

// out dtype dispatch for host launchers
#define PIEH_DISPATCH_DTYPE(code, T, ...)                     \
  do {                                                        \
    if ((code) == PIE_DTYPE_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else { using T = float; __VA_ARGS__; }                    \
  } while (0)

}  // namespace pieh
