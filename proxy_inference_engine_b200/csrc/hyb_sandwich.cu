// Sandwich-norm residual blocks and the grouped, gated output norm of recurrent mixers.
//   sandwich_add_kernel       x[t] += mult * rms_norm(y[t]) * post_w: the sublayer's output (a plain row, or gathered here
//                             from a mixture of experts) passes its own norm on the way INTO the residual; then the optional
//                             re-injection of a looped stack (a saved row and a per-pass vector), and the NEXT sublayer's
//                             input norm h[t] = rms_norm(x[t]) * next_w in the act dtype -- one pass over x per sublayer.
//                             One CTA per token row; y's row and then x's row stay in shared memory between the passes.
//   gated_group_norm_kernel   one warp per (token, group): the group's root mean square, the norm weight and a sigmoid / silu
//                             gate that multiplies either after the norm or before it (then the gated values are normed)
// All sums are fp32 in a fixed order, so a row's result does not depend on what else is in the step.
#include "hyb_common.cuh"

namespace pieh {

template <typename AT>
__global__ void __launch_bounds__(256) sandwich_add_kernel(float* x, const float* y, const pieh_mix_sum mix,
                                                           const float* post_w, float mult, const float* add_rows,
                                                           const float* add_vec, AT* h, const float* next_w, float eps,
                                                           int W) {
  extern __shared__ float row[];
  __shared__ float red[33];
  pdl_sync();
  const int t = blockIdx.x;
  const bool has_y = y != nullptr || mix.parts != nullptr;
  float inv_y = 0.f;
  if (has_y) {
    float ss = 0.f;
    if (mix.parts) {
      float sg = 1.f;
      if (mix.shared && mix.shared_gate) sg = 1.f / (1.f + expf(-mix.shared_gate[(size_t)t * mix.gate_ld]));
      for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v = 0.f;
        for (int k = 0; k < mix.top; ++k)   // choice order: the sum does not depend on how the slots were handed out
          v = fmaf(mix.part_w[(size_t)t * mix.top + k], mix.parts[(size_t)mix.part_row[(size_t)t * mix.top + k] * W + c], v);
        if (mix.shared) v = fmaf(sg, mix.shared[(size_t)t * W + c], v);
        row[c] = v;
        ss = fmaf(v, v, ss);
      }
    } else {
      for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = y[(size_t)t * W + c];
        row[c] = v;
        ss = fmaf(v, v, ss);
      }
    }
    ss = block_sum(ss, red);
    inv_y = mult / sqrtf(ss / (float)W + eps);
  }
  float sx = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = x[(size_t)t * W + c];
    if (has_y) v = fmaf(row[c] * inv_y, post_w[c], v);
    if (add_rows) v += add_rows[(size_t)t * W + c];
    if (add_vec) v += add_vec[c];
    if (has_y || add_rows || add_vec) x[(size_t)t * W + c] = v;
    row[c] = v;            // each thread rewrites only the entries it read
    sx = fmaf(v, v, sx);
  }
  if (!h || !next_w) return;
  sx = block_sum(sx, red);
  const float inv_x = 1.f / sqrtf(sx / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) elem<AT>::store(h + (size_t)t * W + c, row[c] * inv_x * next_w[c]);
}

__device__ __forceinline__ float gate_value(int fn, float g) {
  return fn == 1 ? 1.f / (1.f + expf(-g)) : fn == 2 ? silu_f(g) : 1.f;
}

template <typename OT>
__global__ void gated_group_norm_kernel(OT* out, const float* x, long long x_ld, const float* gate, long long gate_ld,
                                        const float* w, int groups, int gs, float eps, int gate_fn, int gate_first, int T) {
  pdl_sync();
  const long long wi = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wi >= (long long)T * groups) return;
  const int t = (int)(wi / groups), g = (int)(wi - (long long)t * groups);
  const float* xr = x + (size_t)t * x_ld + (size_t)g * gs;
  const float* gr = gate ? gate + (size_t)t * gate_ld + (size_t)g * gs : nullptr;
  const bool pre = gate_first && gr && gate_fn;
  float ss = 0.f;
  for (int c = lane; c < gs; c += 32) {
    float v = xr[c];
    if (pre) v *= gate_value(gate_fn, gr[c]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)gs + eps);
  OT* o = out + ((size_t)t * groups + g) * gs;
  for (int c = lane; c < gs; c += 32) {
    float v = xr[c];
    const float gv = gr && gate_fn ? gate_value(gate_fn, gr[c]) : 1.f;
    v = pre ? v * gv * inv * w[(size_t)g * gs + c] : v * inv * w[(size_t)g * gs + c] * gv;
    elem<OT>::store(o + c, v);
  }
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_sandwich_add(float* x, const float* y, const pieh_mix_sum* mix, const float* post_w, float mult,
                                 const float* add_rows, const float* add_vec, void* h, int h_dtype, const float* next_w,
                                 float eps, int T, int W, void* stream) {
  if (!x) return PIE_ENULL;
  const bool has_mix = mix && mix->parts;
  if ((y || has_mix) && !post_w) return PIE_ENULL;
  if (has_mix && (!mix->part_row || !mix->part_w || mix->top < 1)) return PIE_ENULL;
  if (T < 0 || W < 1 || (size_t)W * 4 > 200 * 1024) return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  pieh_mix_sum m = {};
  if (has_mix) m = *mix;
  const size_t smem = (size_t)W * 4;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(sandwich_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(sandwich_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  count_launch();
  PIEH_DISPATCH_DTYPE(h_dtype, AT, launch_k(sandwich_add_kernel<AT>, dim3(T), dim3(256), smem, (cudaStream_t)stream, x, y, m,
                                            post_w, mult, add_rows, add_vec, (AT*)h, next_w, eps, W));
  return status_of(cudaGetLastError());
}

extern "C" int pieh_gated_group_norm(void* out, int out_dtype, const float* x, long long x_ld, const float* gate,
                                     long long gate_ld, const float* w, int groups, int group_size, float eps, int gate_fn,
                                     int gate_first, int T, void* stream) {
  if (!out || !x || !w || (gate_fn && !gate)) return PIE_ENULL;
  if (T < 0 || groups < 1 || group_size < 1 || gate_fn < 0 || gate_fn > 2) return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  const long long warps = (long long)T * groups;
  count_launch();
  PIEH_DISPATCH_DTYPE(out_dtype, OT, launch_k(gated_group_norm_kernel<OT>, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0,
                                              (cudaStream_t)stream, (OT*)out, x, x_ld, gate, gate_ld, w, groups, group_size,
                                              eps, gate_fn, gate_first, T));
  return status_of(cudaGetLastError());
}
