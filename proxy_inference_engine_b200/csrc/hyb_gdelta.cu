// Generalized delta rule over ragged steps: a matrix state S [dk, dv] per (sequence, head) in fp32, carried in a slot.
//   per token:  p = u^T S;   S <- diag(w) S - (a * u) p + k v^T;   o = S^T r
// with a decay w per key channel, a removal rate a per key channel and the unit key u = k / sqrt(|k|^2 + eps): the old
// content is forgotten channel by channel and, on top of that, erased along the direction of the current key.
// gdelta_prepare_kernel  per (token, head): w = exp(-c sigmoid(decay logits)), a = sigmoid(. + bias), u and a * u
// gdelta_scan_kernel     the recurrence.  A column of S lives in the registers of R adjacent lanes (RPT rows each), so a
//                        token costs 4 RPT multiply-adds and two log2(R)-step shuffle chains per thread and no barrier; the
//                        token's five key-sized vectors and its value entries come through shared memory a chunk of tokens
//                        at a time, cp.async filling one buffer while the recurrence walks the other
// Everything here is fp32.
#include <stdlib.h>

#include "hyb_common.cuh"

namespace pieh {

// grid (T, H)
__global__ void __launch_bounds__(128) gdelta_prepare_kernel(float* decay, float* u, float* au, const float* proj,
                                                             long long ld, const float* dl, long long dl_ld,
                                                             const pieh_gdelta d) {
  __shared__ float red[33];
  pdl_sync();
  const int t = blockIdx.x, h = blockIdx.y;
  const int dk = d.dk;
  const float* kr = proj + (size_t)t * ld + d.k_off + (size_t)h * dk;
  const float* ar = proj + (size_t)t * ld + d.a_off + (size_t)h * dk;
  const float* lr = dl + (size_t)t * dl_ld + (size_t)h * dk;
  float ss = 0.f;
  for (int c = threadIdx.x; c < dk; c += blockDim.x) ss = fmaf(kr[c], kr[c], ss);
  const float inv = 1.f / sqrtf(block_sum(ss, red) + d.key_eps);
  const size_t o = ((size_t)t * d.H + h) * dk;
  for (int c = threadIdx.x; c < dk; c += blockDim.x) {
    const float uu = kr[c] * inv;
    const float a = 1.f / (1.f + expf(-(ar[c] + (d.a_bias ? d.a_bias[(size_t)h * dk + c] : 0.f))));
    decay[o + c] = expf(-d.decay_scale / (1.f + expf(-lr[c])));
    u[o + c] = uu;
    au[o + c] = a * uu;
  }
}

constexpr int kGdThreads = 128;

__device__ __forceinline__ void gd_cp_async(float* smem_dst, const float* gsrc, int bytes) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gsrc) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gsrc) : "memory");
}

// grid (ceil(dv / cols), H, sequences); chunk: tokens per shared-memory buffer
template <int RPT>
__global__ void __launch_bounds__(kGdThreads) gdelta_scan_kernel(float* o, const float* proj, long long ld,
                                                                 const float* decay, const float* u, const float* au,
                                                                 const pieh_gdelta d, const pieh_batch b, int R, int chunk) {
  extern __shared__ __align__(16) float sm[];
  pdl_sync();
  const int cols = kGdThreads / R;
  const int h = blockIdx.y, i = blockIdx.z;
  const int start = b.seq_start[i], n = b.seq_len[i], ctx = b.seq_ctx[i];
  const int rl = threadIdx.x % R, cl = threadIdx.x / R;
  const int j = blockIdx.x * cols + cl;           // column of S (feature of v)
  const bool col_ok = j < d.dv;
  const int dk = d.dk, dv = d.dv;
  // one buffer: per token [w | u | a u | k | r] (dk each), then the chunk's value entries [chunk, cols]
  const int tok_floats = 5 * dk;
  const int buf_floats = chunk * (tok_floats + cols);
  float* S_g = d.state + (((size_t)b.seq_slot[i] * d.H + h) * dk) * dv;
  float S[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int row = r * R + rl;   // rows are dealt round-robin to the R lanes: neighbouring lanes read neighbouring banks
    S[r] = (ctx > 0 && col_ok && row < dk) ? S_g[(size_t)row * dv + j] : 0.f;
  }
  // 16-byte copies need every source 16-byte aligned: whole multiples of 4 floats everywhere a row starts
  const bool vec = (dk & 3) == 0 && (ld & 3) == 0 && (d.k_off & 3) == 0 && (d.r_off & 3) == 0 &&
                   (reinterpret_cast<uintptr_t>(proj) & 15) == 0 && (reinterpret_cast<uintptr_t>(decay) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(u) & 15) == 0 && (reinterpret_cast<uintptr_t>(au) & 15) == 0;
  auto fill = [&](int which, int c0) {
    float* base = sm + which * buf_floats;
    float* vs = base + chunk * tok_floats;
    const int nc = min(chunk, n - c0);
    const int step = vec ? 4 : 1, per = dk / step;
    for (int e = threadIdx.x; e < nc * per; e += kGdThreads) {
      const int tt = e / per, r = (e - tt * per) * step;
      const size_t row = (size_t)(start + c0 + tt);
      const size_t s3 = (row * d.H + h) * dk + r;
      float* dst = base + tt * tok_floats + r;
      gd_cp_async(dst, decay + s3, 4 * step);
      gd_cp_async(dst + dk, u + s3, 4 * step);
      gd_cp_async(dst + 2 * dk, au + s3, 4 * step);
      gd_cp_async(dst + 3 * dk, proj + row * ld + d.k_off + (size_t)h * dk + r, 4 * step);
      gd_cp_async(dst + 4 * dk, proj + row * ld + d.r_off + (size_t)h * dk + r, 4 * step);
    }
    for (int e = threadIdx.x; e < nc * cols; e += kGdThreads) {
      const int tt = e / cols, c = e - tt * cols;
      const int jj = min(blockIdx.x * cols + c, dv - 1);
      gd_cp_async(vs + e, proj + (size_t)(start + c0 + tt) * ld + d.v_off + (size_t)h * dv + jj, 4);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float out_prev = 0.f;   // this lane's share of the last token's read-out, not yet summed over the R lanes
  int row_prev = -1;
  fill(0, 0);
  for (int c0 = 0, which = 0; c0 < n; c0 += chunk, which ^= 1) {
    const int nc = min(chunk, n - c0);
    if (c0 + chunk < n) {
      fill(which ^ 1, c0 + chunk);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* base = sm + which * buf_floats;
    const float* vs = base + chunk * tok_floats;
    for (int tt = 0; tt < nc; ++tt) {
      const float* tk = base + tt * tok_floats + rl;
      float pp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < RPT; ++r)
        if (r * R + rl < dk) pp[r & 3] = fmaf(S[r], tk[dk + r * R], pp[r & 3]);
      float p = (pp[0] + pp[1]) + (pp[2] + pp[3]);
      // the read-out of the PREVIOUS token is reduced over the R lanes together with this token's projection: two
      // independent shuffle chains instead of two in a row on the recurrence's critical path
      for (int off = 1; off < R; off <<= 1) {
        p += __shfl_xor_sync(0xffffffffu, p, off);
        out_prev += __shfl_xor_sync(0xffffffffu, out_prev, off);
      }
      if (row_prev >= 0 && rl == 0 && col_ok) o[((size_t)row_prev * d.H + h) * dv + j] = out_prev;
      const float vj = vs[tt * cols + cl];
      float oo[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        if (r * R + rl < dk) {
          const float* e = tk + r * R;
          S[r] = fmaf(e[0], S[r], fmaf(e[3 * dk], vj, -e[2 * dk] * p));
          oo[r & 3] = fmaf(S[r], e[4 * dk], oo[r & 3]);
        }
      }
      out_prev = (oo[0] + oo[1]) + (oo[2] + oo[3]);
      row_prev = start + c0 + tt;
    }
    __syncthreads();   // everyone is done with this buffer before the next fill overwrites it
  }
  for (int off = 1; off < R; off <<= 1) out_prev += __shfl_xor_sync(0xffffffffu, out_prev, off);
  if (row_prev >= 0 && rl == 0 && col_ok) o[((size_t)row_prev * d.H + h) * dv + j] = out_prev;
  if (col_ok) {
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int row = r * R + rl;
      if (row < dk) S_g[(size_t)row * dv + j] = S[r];
    }
  }
}

constexpr int kFixChunk = 16;   // tokens per shared-memory buffer of the fixed-size kernels

// The same recurrence with the key size fixed at compile time.  A lane owns Q runs of four neighbouring state rows (R = DK / 4 Q
// lanes per column), so a token's five key-sized vectors arrive as 5 Q 16-byte shared-memory loads with constant offsets and
// nothing is predicated; a CTA is COLS columns wide (R COLS threads).  With few rows per lane a column's work is spread over
// many warps: one sequence's heads then fill every scheduler with several warps whose shuffle and shared-memory latencies
// overlap, where one warp per scheduler would sit out each of them.  Needs every row start 16-byte aligned.
template <int DK, int Q, int COLS>
__global__ void __launch_bounds__(DK / (4 * Q) * COLS) gdelta_scan_fixed_kernel(float* o, const float* proj, long long ld,
                                                                                const float* decay, const float* u,
                                                                                const float* au, const pieh_gdelta d,
                                                                                const pieh_batch b) {
  constexpr int R = DK / (4 * Q), NT = R * COLS, chunk = kFixChunk;
  constexpr int tok_floats = 5 * DK, buf_floats = chunk * (tok_floats + COLS);
  static_assert(R >= 1 && R <= 32 && (R & (R - 1)) == 0 && NT % 32 == 0, "the lanes of a column sit in one warp");
  extern __shared__ __align__(16) float sm[];
  pdl_sync();
  const int h = blockIdx.y, i = blockIdx.z;
  const int start = b.seq_start[i], n = b.seq_len[i], ctx = b.seq_ctx[i];
  const int rl = threadIdx.x % R, cl = threadIdx.x / R;
  const int j = blockIdx.x * COLS + cl;           // column of S (feature of v)
  const int dv = d.dv;
  const bool col_ok = j < dv;
  float* S_g = d.state + (((size_t)b.seq_slot[i] * d.H + h) * DK) * dv;
  float S[4 * Q];   // S[4 q + e] is state row q * 4 R + 4 rl + e
#pragma unroll
  for (int q = 0; q < Q; ++q)
#pragma unroll
    for (int e = 0; e < 4; ++e)
      S[4 * q + e] = (ctx > 0 && col_ok) ? S_g[(size_t)(q * 4 * R + 4 * rl + e) * dv + j] : 0.f;
  auto fill = [&](int which, int c0) {
    float* base = sm + which * buf_floats;
    float* vs = base + chunk * tok_floats;
    const int nc = min(chunk, n - c0);
    constexpr int per = DK / 4;
    for (int e = threadIdx.x; e < nc * per; e += NT) {
      const int tt = e / per, r = (e - tt * per) * 4;
      const size_t row = (size_t)(start + c0 + tt);
      const size_t s3 = (row * d.H + h) * DK + r;
      float* dst = base + tt * tok_floats + r;
      gd_cp_async(dst, decay + s3, 16);
      gd_cp_async(dst + DK, u + s3, 16);
      gd_cp_async(dst + 2 * DK, au + s3, 16);
      gd_cp_async(dst + 3 * DK, proj + row * ld + d.k_off + (size_t)h * DK + r, 16);
      gd_cp_async(dst + 4 * DK, proj + row * ld + d.r_off + (size_t)h * DK + r, 16);
    }
    for (int e = threadIdx.x; e < nc * COLS; e += NT) {
      const int tt = e / COLS, c = e - tt * COLS;
      const int jj = min(blockIdx.x * COLS + c, dv - 1);
      gd_cp_async(vs + e, proj + (size_t)(start + c0 + tt) * ld + d.v_off + (size_t)h * dv + jj, 4);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float out_prev = 0.f;
  int row_prev = -1;
  fill(0, 0);
  for (int c0 = 0, which = 0; c0 < n; c0 += chunk, which ^= 1) {
    const int nc = min(chunk, n - c0);
    if (c0 + chunk < n) {
      fill(which ^ 1, c0 + chunk);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* base = sm + which * buf_floats;
    const float* vs = base + chunk * tok_floats;
#pragma unroll 2
    for (int tt = 0; tt < nc; ++tt) {
      const float4* t4 = reinterpret_cast<const float4*>(base + tt * tok_floats) + rl;   // + q R: run q; + DK / 4: next vector
      float4 uu[Q], ww[Q], aa[Q], kk[Q], rr[Q];
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        ww[q] = t4[q * R]; uu[q] = t4[DK / 4 + q * R]; aa[q] = t4[2 * (DK / 4) + q * R];
        kk[q] = t4[3 * (DK / 4) + q * R]; rr[q] = t4[4 * (DK / 4) + q * R];
      }
      float pp[Q];
#pragma unroll
      for (int q = 0; q < Q; ++q)
        pp[q] = fmaf(S[4 * q + 3], uu[q].w, fmaf(S[4 * q + 2], uu[q].z, fmaf(S[4 * q + 1], uu[q].y, S[4 * q] * uu[q].x)));
      float p = pp[0];
#pragma unroll
      for (int q = 1; q < Q; ++q) p += pp[q];
      // the read-out of the PREVIOUS token is reduced over the R lanes together with this token's projection
#pragma unroll
      for (int off = 1; off < R; off <<= 1) {
        p += __shfl_xor_sync(0xffffffffu, p, off);
        out_prev += __shfl_xor_sync(0xffffffffu, out_prev, off);
      }
      if (row_prev >= 0 && rl == 0 && col_ok) o[((size_t)row_prev * d.H + h) * dv + j] = out_prev;
      const float vj = vs[tt * COLS + cl];
      float oo[Q];
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        S[4 * q] = fmaf(ww[q].x, S[4 * q], fmaf(kk[q].x, vj, -aa[q].x * p));
        S[4 * q + 1] = fmaf(ww[q].y, S[4 * q + 1], fmaf(kk[q].y, vj, -aa[q].y * p));
        S[4 * q + 2] = fmaf(ww[q].z, S[4 * q + 2], fmaf(kk[q].z, vj, -aa[q].z * p));
        S[4 * q + 3] = fmaf(ww[q].w, S[4 * q + 3], fmaf(kk[q].w, vj, -aa[q].w * p));
        oo[q] = fmaf(S[4 * q + 3], rr[q].w, fmaf(S[4 * q + 2], rr[q].z, fmaf(S[4 * q + 1], rr[q].y, S[4 * q] * rr[q].x)));
      }
      out_prev = oo[0];
#pragma unroll
      for (int q = 1; q < Q; ++q) out_prev += oo[q];
      row_prev = start + c0 + tt;
    }
    __syncthreads();
  }
#pragma unroll
  for (int off = 1; off < R; off <<= 1) out_prev += __shfl_xor_sync(0xffffffffu, out_prev, off);
  if (row_prev >= 0 && rl == 0 && col_ok) o[((size_t)row_prev * d.H + h) * dv + j] = out_prev;
  if (col_ok) {
#pragma unroll
    for (int q = 0; q < Q; ++q)
#pragma unroll
      for (int e = 0; e < 4; ++e) S_g[(size_t)(q * 4 * R + 4 * rl + e) * dv + j] = S[4 * q + e];
  }
}

template <int DK, int Q, int COLS>
static cudaError_t launch_gdelta_fixed(float* o, const float* proj, long long ld, const float* decay, const float* u,
                                       const float* au, const pieh_gdelta& d, const pieh_batch& b, cudaStream_t st) {
  constexpr int NT = DK / (4 * Q) * COLS;
  constexpr size_t smem = (size_t)2 * kFixChunk * (5 * DK + COLS) * 4;
  static bool opted = false;
  if (smem > 48 * 1024 && !opted) {
    cudaFuncSetAttribute(gdelta_scan_fixed_kernel<DK, Q, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    opted = true;
  }
  return launch_k(gdelta_scan_fixed_kernel<DK, Q, COLS>, dim3((d.dv + COLS - 1) / COLS, d.H, b.n_seq), dim3(NT), smem, st, o,
                  proj, ld, decay, u, au, d, b);
}

static bool gdelta_ok(const pieh_gdelta* d) {
  return d && d->H > 0 && d->dk > 0 && d->dv > 0 && d->dk <= 512 && d->dv <= 65535 && d->r_off >= 0 && d->k_off >= 0 &&
         d->v_off >= 0 && d->a_off >= 0 && d->state && d->key_eps >= 0.f;
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_gdelta_prepare(float* decay, float* u, float* au, const float* proj, long long ld,
                                   const float* decay_logits, long long dl_ld, const pieh_gdelta* d, int T, void* stream) {
  if (!decay || !u || !au || !proj || !decay_logits || !d) return PIE_ENULL;
  if (!gdelta_ok(d) || T < 0 || d->H > 65535) return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  count_launch();
  return status_of(launch_k(gdelta_prepare_kernel, dim3(T, d->H), dim3(128), 0, (cudaStream_t)stream, decay, u, au, proj, ld,
                            decay_logits, dl_ld, *d));
}

extern "C" int pieh_gdelta_scan(float* o, const float* proj, long long ld, const float* decay, const float* u,
                                const float* au, const pieh_gdelta* d, const pieh_batch* b, void* stream) {
  if (!o || !proj || !decay || !u || !au || !d || !b) return PIE_ENULL;
  if (!gdelta_ok(d) || d->H > 65535 || b->n_seq > 65535) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  const bool aligned = (ld & 3) == 0 && (d->k_off & 3) == 0 && (d->r_off & 3) == 0 &&
                       ((reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(decay) |
                         reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(au)) & 15) == 0;
  static const bool generic_only = [] { const char* e = getenv("PIE_HYBRID_NO_FIXED_SCAN"); return e && e[0] == '1'; }();
  if (aligned && !generic_only && (d->dk == 32 || d->dk == 64 || d->dk == 128)) {
    count_launch();
    cudaStream_t st = (cudaStream_t)stream;
    // measured at dk = dv = 128, 16 heads, one 4096-row portion: 4 / 8 / 16 rows per lane 1.35 / 1.18 / 1.24 ms
    if (d->dk == 128) return status_of(launch_gdelta_fixed<128, 2, 16>(o, proj, ld, decay, u, au, *d, *b, st));
    return status_of(d->dk == 32 ? launch_gdelta_fixed<32, 1, 16>(o, proj, ld, decay, u, au, *d, *b, st)
                     : d->dk == 64 ? launch_gdelta_fixed<64, 1, 16>(o, proj, ld, decay, u, au, *d, *b, st)
                                   : launch_gdelta_fixed<128, 1, 16>(o, proj, ld, decay, u, au, *d, *b, st));
  }
  constexpr int RPT = 16;            // rows of a state column per lane
  int R = 1;
  while (R * RPT < d->dk) R <<= 1;   // lanes per column, a power of two <= 32
  const int cols = kGdThreads / R;
  // tokens per buffer: 16 where two buffers fit the shared memory a CTA may have, fewer for very wide keys
  int chunk = 16;
  while (chunk > 1 && (size_t)2 * chunk * (5 * d->dk + cols) * 4 > 160 * 1024) chunk >>= 1;
  const size_t smem = (size_t)2 * chunk * (5 * d->dk + cols) * 4;
  static bool opted = false;
  if (smem > 48 * 1024 && !opted) {
    cudaFuncSetAttribute(gdelta_scan_kernel<RPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    opted = true;
  }
  count_launch();
  return status_of(launch_k(gdelta_scan_kernel<RPT>, dim3((d->dv + cols - 1) / cols, d->H, b->n_seq), dim3(kGdThreads), smem,
                            (cudaStream_t)stream, o, proj, ld, decay, u, au, *d, *b, R, chunk));
}
