// Mixture-of-experts routing and the plan of the grouped products.
//   moe_route_kernel   one warp per token.  softmax_top: the largest logits, weights = softmax over the chosen logits.
//                      Otherwise: sigmoid scores, group scores (sum of a group's two largest), the best groups
//                      stay eligible, the `top` largest eligible scores are chosen (ties: lower index) with weight
//                      score * scale; it also counts the tokens of every expert
//   moe_plan_kernel    one CTA: prefix sums of the counts -> every (token, choice) pair gets a SLOT in its expert's run,
//                      and the runs are cut into tiles of <= 64 and <= 128 slots for the grouped matrix products
//                      (pieh_moe_linear, hyb_linear.cu).  The order of the pairs inside a run is whatever the atomics
//                      give; every slot is computed on its own and the pairs are summed per token in choice order
//                      (pieh_postnorm_add), so the result does not depend on it.
#include "hyb_common.cuh"

namespace pieh {

constexpr int kMaxExperts = 1024, kMaxTop = 32;

__global__ void __launch_bounds__(32) moe_route_kernel(const float* z, long long ld, const pieh_moe_plan p) {
  __shared__ float s[kMaxExperts];
  __shared__ float gsc[kMaxExperts];
  __shared__ unsigned char ok[kMaxExperts];   // per group: eligible
  pdl_sync();
  const int t = blockIdx.x, lane = threadIdx.x;
  const int E = p.E, per = E / p.n_groups;
  if (p.softmax_top) {
    // the `top` largest logits, weighted by the softmax over those logits alone (ties: lower index)
    __shared__ float chosen[kMaxTop];
    for (int e = lane; e < E; e += 32) s[e] = z[(size_t)t * ld + e];
    __syncwarp();
    for (int r = 0; r < p.top; ++r) {
      float bv = -INFINITY;
      int bi = E;
      for (int i = lane; i < E; i += 32)
        if (s[i] > bv) { bv = s[i]; bi = i; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      __syncwarp();
      if (lane == 0) {
        const int ee = bi < E ? bi : 0;
        chosen[r] = bi < E ? bv : -INFINITY;
        p.pair_slot[(size_t)t * p.top + r] = ee;
        atomicAdd(&p.counters[ee], 1);
        if (bi < E) s[ee] = -INFINITY;   // taken
      }
      __syncwarp();
    }
    if (lane == 0) {
      float sum = 0.f;
      for (int r = 0; r < p.top; ++r) sum += expf(chosen[r] - chosen[0]);   // chosen[0] is the largest
      for (int r = 0; r < p.top; ++r) p.pair_w[(size_t)t * p.top + r] = expf(chosen[r] - chosen[0]) / sum * p.scale;
    }
    return;
  }
  for (int e = lane; e < E; e += 32) s[e] = 1.f / (1.f + expf(-z[(size_t)t * ld + e]));
  __syncwarp();
  for (int g = lane; g < p.n_groups; g += 32) {
    float a = -1.f, b = -1.f;   // scores are in (0, 1)
    for (int e = g * per; e < (g + 1) * per; ++e) {
      const float v = s[e];
      if (v > a) { b = a; a = v; } else if (v > b) b = v;
    }
    gsc[g] = per > 1 ? a + b : a;
    ok[g] = 0;
  }
  __syncwarp();
  // argmax rounds over the warp: value descending, index ascending
  auto pick = [&](const float* val, int n, auto usable) {
    float bv = -2.f;
    int bi = n;
    for (int i = lane; i < n; i += 32)
      if (usable(i) && val[i] > bv) { bv = val[i]; bi = i; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    return bi;
  };
  for (int r = 0; r < p.keep_groups; ++r) {
    const int g = pick(gsc, p.n_groups, [&](int i) { return ok[i] == 0; });
    __syncwarp();
    if (lane == 0 && g < p.n_groups) ok[g] = 1;
    __syncwarp();
  }
  for (int r = 0; r < p.top; ++r) {
    const int e = pick(s, E, [&](int i) { return ok[i / per] == 1 && s[i] >= 0.f; });
    __syncwarp();
    if (lane == 0) {
      const int ee = e < E ? e : 0;   // fewer eligible experts than `top` cannot happen with a valid configuration
      p.pair_slot[(size_t)t * p.top + r] = ee;            // expert id for now; the plan turns it into a slot
      p.pair_w[(size_t)t * p.top + r] = e < E ? s[ee] * p.scale : 0.f;
      atomicAdd(&p.counters[ee], 1);
      if (e < E) s[ee] = -1.f;                            // taken
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(1024) moe_plan_kernel(const pieh_moe_plan p, int P) {
  __shared__ int off[kMaxExperts + 1], cur[kMaxExperts], t64[kMaxExperts + 1], t128[kMaxExperts + 1];
  pdl_sync();
  const int E = p.E;
  if (threadIdx.x == 0) {
    int o = 0, a = 0, b = 0;
    for (int e = 0; e < E; ++e) {
      const int c = p.counters[e];
      off[e] = o; t64[e] = a; t128[e] = b;
      o += c; a += (c + 63) / 64; b += (c + 127) / 128;
    }
    off[E] = o; t64[E] = a; t128[E] = b;
    p.tiles64[0] = a;
    p.tiles128[0] = b;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) cur[e] = 0;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int c = off[e + 1] - off[e];
    for (int r = 0, i = t64[e]; r < c; r += 64, ++i) {
      p.tiles64[1 + 3 * i] = e; p.tiles64[2 + 3 * i] = off[e] + r; p.tiles64[3 + 3 * i] = min(64, c - r);
    }
    for (int r = 0, i = t128[e]; r < c; r += 128, ++i) {
      p.tiles128[1 + 3 * i] = e; p.tiles128[2 + 3 * i] = off[e] + r; p.tiles128[3 + 3 * i] = min(128, c - r);
    }
  }
  for (int q = threadIdx.x; q < P; q += blockDim.x) {
    const int e = p.pair_slot[q];
    const int slot = off[e] + atomicAdd(&cur[e], 1);
    p.pair_slot[q] = slot;
    p.slot_row[slot] = q / p.top;
    p.slot_expert[slot] = e;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) p.counters[e] = 0;   // ready for the next step
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_moe_route(const float* z, long long ld, const pieh_moe_plan* p, int T, void* stream) {
  if (!z || !p || !p->slot_row || !p->slot_expert || !p->pair_slot || !p->pair_w || !p->tiles64 || !p->tiles128 ||
      !p->counters)
    return PIE_ENULL;
  if (T < 0 || p->E < 1 || p->E > kMaxExperts || p->top < 1 || p->top > kMaxTop || p->n_groups < 1 ||
      p->E % p->n_groups != 0 || p->keep_groups < 1 || p->keep_groups > p->n_groups ||
      (long long)p->keep_groups * (p->E / p->n_groups) < p->top)
    return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  count_launch(2);
  cudaError_t e = launch_k(moe_route_kernel, dim3(T), dim3(32), 0, st, z, ld, *p);
  if (e == cudaSuccess) e = launch_k(moe_plan_kernel, dim3(1), dim3(1024), 0, st, *p, T * p->top);
  return status_of(e);
}
