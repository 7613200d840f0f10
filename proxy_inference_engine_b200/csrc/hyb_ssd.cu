// Selective state-space layer with one scalar decay per head and token (the "state-space duality" form) over ragged steps.
//   per token and head:  S <- exp(-exp(A_log) dt) S + dt B x^T   (S [N, P], fp32, in the sequence's slot);   y = S^T C + D x
// ssd_prepare_kernel   per token: causal convolution over time (+ bias) and silu on the channels [x | B | C] -- rows before the
//                      step come from the sequence's history of taps - 1 inputs, rows before the sequence are zero -- and per
//                      head dt = softplus(logit + bias), decay = exp(-exp(A_log) dt)
// ssd_advance_kernel   afterwards: every sequence's history moves past this step's rows
// ssd_scan_kernel      the recurrence.  A column of S (one feature of x) lives in the registers of R adjacent lanes (RPT state
//                      rows each): a token costs 2 RPT multiply-adds and one log2(R)-step shuffle chain per thread, deferred by
//                      one token so that it is off the critical path; B, C, x and the two scalars of a chunk of tokens are
//                      staged in shared memory by cp.async, one buffer filling while the other is walked
// Everything here is fp32.
#include <stdlib.h>

#include "hyb_common.cuh"

namespace pieh {

constexpr int kSsdMaxTaps = 8;

__global__ void __launch_bounds__(256) ssd_prepare_kernel(float* xbc, float* dtd, const float* proj, long long ld,
                                                          const pieh_ssd s, const pieh_batch b) {
  pdl_sync();
  const int t = blockIdx.x;
  const int i = b.tok_seq[t], start = b.seq_start[i], ctx = b.seq_ctx[i], slot = b.seq_slot[i];
  const int j = t - start;
  const int C = s.H * s.P + 2 * s.G * s.N, taps = s.taps;
  const float* hist = taps > 1 ? s.conv_state + (size_t)slot * (taps - 1) * C : nullptr;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = s.conv_b ? s.conv_b[c] : 0.f;
    for (int r = taps - 1; r >= 0; --r) {   // oldest input first
      float x;
      if (r <= j) x = proj[(size_t)(t - r) * ld + s.xbc_off + c];
      else {
        const int back = r - j;             // 1 .. taps - 1 tokens before this step
        x = ctx - back >= 0 ? hist[(size_t)(taps - 1 - back) * C + c] : 0.f;
      }
      acc = fmaf(s.conv_w[(size_t)c * taps + (taps - 1 - r)], x, acc);
    }
    xbc[(size_t)t * C + c] = silu_f(acc);
  }
  for (int h = threadIdx.x; h < s.H; h += blockDim.x) {
    const float dt = softplus_f(proj[(size_t)t * ld + s.dt_off + h] + s.dt_bias[h]);
    dtd[((size_t)t * s.H + h) * 2] = dt;
    dtd[((size_t)t * s.H + h) * 2 + 1] = expf(-expf(s.A_log[h]) * dt);
  }
}

__global__ void ssd_advance_kernel(const float* proj, long long ld, const pieh_ssd s, const pieh_batch b) {
  pdl_sync();
  const int i = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int C = s.H * s.P + 2 * s.G * s.N, taps = s.taps;
  if (c >= C) return;
  const int start = b.seq_start[i], n = b.seq_len[i], ctx = b.seq_ctx[i];
  float* hist = s.conv_state + (size_t)b.seq_slot[i] * (taps - 1) * C;
  float nv[kSsdMaxTaps];
  for (int jj = 0; jj < taps - 1; ++jj) {
    const int p = ctx + n - (taps - 1) + jj;   // position this entry has to hold afterwards
    float x = 0.f;
    if (p >= ctx) x = proj[(size_t)(start + p - ctx) * ld + s.xbc_off + c];
    else if (p >= 0) x = hist[(size_t)(p - ctx + taps - 1) * C + c];
    nv[jj] = x;
  }
  for (int jj = 0; jj < taps - 1; ++jj) hist[(size_t)jj * C + c] = nv[jj];
}

constexpr int kSsdThreads = 128, kSsdChunk = 16;

__device__ __forceinline__ void ssd_cp_async(float* smem_dst, const float* gsrc, int bytes) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gsrc) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gsrc) : "memory");
}

// grid (ceil(P / cols), H, sequences)
template <int RPT>
__global__ void __launch_bounds__(kSsdThreads) ssd_scan_kernel(float* y, const float* xbc, const float* dtd, const pieh_ssd s,
                                                               const pieh_batch b, int R) {
  extern __shared__ __align__(16) float sm[];
  pdl_sync();
  const int cols = kSsdThreads / R;
  const int h = blockIdx.y, i = blockIdx.z;
  const int g = h / (s.H / s.G);
  const int start = b.seq_start[i], n = b.seq_len[i], ctx = b.seq_ctx[i];
  const int rl = threadIdx.x % R, cl = threadIdx.x / R;
  const int j = blockIdx.x * cols + cl;           // column of S (feature of x)
  const bool col_ok = j < s.P;
  const int N = s.N, P = s.P;
  const int C = s.H * P + 2 * s.G * N;
  const int offB = s.H * P + g * N, offC = s.H * P + s.G * N + g * N;
  // one buffer: per token [B | C] (N each), then [chunk, cols] entries of x, then [chunk, 2] (dt, decay)
  const int buf_floats = kSsdChunk * (2 * N + cols + 2);
  float* S_g = s.state + (((size_t)b.seq_slot[i] * s.H + h) * N) * P;
  float S[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int row = r * R + rl;
    S[r] = (ctx > 0 && col_ok && row < N) ? S_g[(size_t)row * P + j] : 0.f;
  }
  const float Dh = s.D ? s.D[h] : 0.f;
  const bool vec = (N & 3) == 0 && (C & 3) == 0 && ((s.H * P) & 3) == 0 && (reinterpret_cast<uintptr_t>(xbc) & 15) == 0;
  auto fill = [&](int which, int c0) {
    float* bc = sm + which * buf_floats;
    float* xs = bc + kSsdChunk * 2 * N;
    float* sc = xs + kSsdChunk * cols;
    const int nc = min(kSsdChunk, n - c0);
    const int step = vec ? 4 : 1, per = N / step;
    for (int e = threadIdx.x; e < nc * per; e += kSsdThreads) {
      const int tt = e / per, r = (e - tt * per) * step;
      const float* row = xbc + (size_t)(start + c0 + tt) * C;
      ssd_cp_async(bc + tt * 2 * N + r, row + offB + r, 4 * step);
      ssd_cp_async(bc + tt * 2 * N + N + r, row + offC + r, 4 * step);
    }
    for (int e = threadIdx.x; e < nc * cols; e += kSsdThreads) {
      const int tt = e / cols, c = e - tt * cols;
      const int jj = min(blockIdx.x * cols + c, P - 1);
      ssd_cp_async(xs + e, xbc + (size_t)(start + c0 + tt) * C + (size_t)h * P + jj, 4);
    }
    for (int e = threadIdx.x; e < nc * 2; e += kSsdThreads)
      ssd_cp_async(sc + e, dtd + ((size_t)(start + c0 + (e >> 1)) * s.H + h) * 2 + (e & 1), 4);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float out_prev = 0.f, skip_prev = 0.f;   // last token's read-out (this lane's share) and its D x term
  int row_prev = -1;
  fill(0, 0);
  for (int c0 = 0, which = 0; c0 < n; c0 += kSsdChunk, which ^= 1) {
    const int nc = min(kSsdChunk, n - c0);
    if (c0 + kSsdChunk < n) {
      fill(which ^ 1, c0 + kSsdChunk);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* bc = sm + which * buf_floats;
    const float* xs = bc + kSsdChunk * 2 * N;
    const float* sc = xs + kSsdChunk * cols;
    for (int tt = 0; tt < nc; ++tt) {
      // the previous token's read-out is summed over the R lanes while this token's update runs
      for (int off = 1; off < R; off <<= 1) out_prev += __shfl_xor_sync(0xffffffffu, out_prev, off);
      if (row_prev >= 0 && rl == 0 && col_ok) y[((size_t)row_prev * s.H + h) * P + j] = out_prev + skip_prev;
      const float dt = sc[2 * tt], dec = sc[2 * tt + 1];
      const float xj = xs[tt * cols + cl];
      const float dx = dt * xj;
      const float* Br = bc + tt * 2 * N + rl;
      float oo[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        if (r * R + rl < N) {
          S[r] = fmaf(dec, S[r], dx * Br[r * R]);
          oo[r & 3] = fmaf(S[r], Br[N + r * R], oo[r & 3]);
        }
      }
      out_prev = (oo[0] + oo[1]) + (oo[2] + oo[3]);
      skip_prev = Dh * xj;
      row_prev = start + c0 + tt;
    }
    __syncthreads();   // everyone is done with this buffer before the next fill overwrites it
  }
  for (int off = 1; off < R; off <<= 1) out_prev += __shfl_xor_sync(0xffffffffu, out_prev, off);
  if (row_prev >= 0 && rl == 0 && col_ok) y[((size_t)row_prev * s.H + h) * P + j] = out_prev + skip_prev;
  if (col_ok) {
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int row = r * R + rl;
      if (row < N) S_g[(size_t)row * P + j] = S[r];
    }
  }
}

// The same recurrence with the state size fixed at compile time.  A lane owns Q runs of four neighbouring state rows (R =
// N / 4 Q lanes per column), so B and C of a token arrive as 2 Q 16-byte shared-memory loads with constant offsets; a CTA is
// COLS columns wide (R COLS threads).  Nothing in a token's update waits for a reduction, so few rows per lane and many
// warps per scheduler is the fast shape: the deferred read-out shuffles of one warp hide behind the others' arithmetic.
constexpr int kFixChunk = 16;   // tokens per shared-memory buffer of the fixed-size kernels

template <int N, int Q, int COLS>
__global__ void __launch_bounds__(N / (4 * Q) * COLS) ssd_scan_fixed_kernel(float* y, const float* xbc, const float* dtd,
                                                                            const pieh_ssd s, const pieh_batch b) {
  constexpr int R = N / (4 * Q), NT = R * COLS;
  constexpr int buf_floats = kFixChunk * (2 * N + COLS + 2);
  static_assert(R >= 1 && R <= 32 && (R & (R - 1)) == 0 && NT % 32 == 0, "the lanes of a column sit in one warp");
  extern __shared__ __align__(16) float sm[];
  pdl_sync();
  const int h = blockIdx.y, i = blockIdx.z;
  const int g = h / (s.H / s.G);
  const int start = b.seq_start[i], n = b.seq_len[i], ctx = b.seq_ctx[i];
  const int rl = threadIdx.x % R, cl = threadIdx.x / R;
  const int j = blockIdx.x * COLS + cl;
  const int P = s.P;
  const bool col_ok = j < P;
  const int C = s.H * P + 2 * s.G * N;
  const int offB = s.H * P + g * N, offC = s.H * P + s.G * N + g * N;
  float* S_g = s.state + (((size_t)b.seq_slot[i] * s.H + h) * N) * P;
  float S[4 * Q];   // S[4 q + e] is state row q * 4 R + 4 rl + e
#pragma unroll
  for (int q = 0; q < Q; ++q)
#pragma unroll
    for (int e = 0; e < 4; ++e)
      S[4 * q + e] = (ctx > 0 && col_ok) ? S_g[(size_t)(q * 4 * R + 4 * rl + e) * P + j] : 0.f;
  const float Dh = s.D ? s.D[h] : 0.f;
  auto fill = [&](int which, int c0) {
    float* bc = sm + which * buf_floats;
    float* xs = bc + kFixChunk * 2 * N;
    float* sc = xs + kFixChunk * COLS;
    const int nc = min(kFixChunk, n - c0);
    constexpr int per = N / 4;
    for (int e = threadIdx.x; e < nc * per; e += NT) {
      const int tt = e / per, r = (e - tt * per) * 4;
      const float* row = xbc + (size_t)(start + c0 + tt) * C;
      ssd_cp_async(bc + tt * 2 * N + r, row + offB + r, 16);
      ssd_cp_async(bc + tt * 2 * N + N + r, row + offC + r, 16);
    }
    for (int e = threadIdx.x; e < nc * COLS; e += NT) {
      const int tt = e / COLS, c = e - tt * COLS;
      const int jj = min(blockIdx.x * COLS + c, P - 1);
      ssd_cp_async(xs + e, xbc + (size_t)(start + c0 + tt) * C + (size_t)h * P + jj, 4);
    }
    for (int e = threadIdx.x; e < nc * 2; e += NT)
      ssd_cp_async(sc + e, dtd + ((size_t)(start + c0 + (e >> 1)) * s.H + h) * 2 + (e & 1), 4);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fill(0, 0);
  for (int c0 = 0, which = 0; c0 < n; c0 += kFixChunk, which ^= 1) {
    const int nc = min(kFixChunk, n - c0);
    if (c0 + kFixChunk < n) {
      fill(which ^ 1, c0 + kFixChunk);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* bc = sm + which * buf_floats;
    const float* xs = bc + kFixChunk * 2 * N;
    const float* sc = xs + kFixChunk * COLS;
    // four tokens at a time: their read-outs are summed over the R lanes as four independent shuffle chains, so a chain's
    // latency is paid once per four tokens (the state update itself never waits for a reduction)
    for (int t0 = 0; t0 < nc; t0 += 4) {
      float part[4], skip[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        part[k] = 0.f; skip[k] = 0.f;
        const int tt = t0 + k;
        if (tt < nc) {
          const float4* t4 = reinterpret_cast<const float4*>(bc + tt * 2 * N) + rl;
          const float dt = sc[2 * tt], dec = sc[2 * tt + 1];
          const float xj = xs[tt * COLS + cl];
          const float dx = dt * xj;
#pragma unroll
          for (int q = 0; q < Q; ++q) {
            const float4 Bv = t4[q * R], Cv = t4[N / 4 + q * R];
            S[4 * q] = fmaf(dec, S[4 * q], dx * Bv.x);
            S[4 * q + 1] = fmaf(dec, S[4 * q + 1], dx * Bv.y);
            S[4 * q + 2] = fmaf(dec, S[4 * q + 2], dx * Bv.z);
            S[4 * q + 3] = fmaf(dec, S[4 * q + 3], dx * Bv.w);
            part[k] += fmaf(S[4 * q + 3], Cv.w, fmaf(S[4 * q + 2], Cv.z, fmaf(S[4 * q + 1], Cv.y, S[4 * q] * Cv.x)));
          }
          skip[k] = Dh * xj;
        }
      }
#pragma unroll
      for (int off = 1; off < R; off <<= 1)
#pragma unroll
        for (int k = 0; k < 4; ++k) part[k] += __shfl_xor_sync(0xffffffffu, part[k], off);
      if (rl == 0 && col_ok) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (t0 + k < nc) y[((size_t)(start + c0 + t0 + k) * s.H + h) * P + j] = part[k] + skip[k];
      }
    }
    __syncthreads();
  }
  if (col_ok) {
#pragma unroll
    for (int q = 0; q < Q; ++q)
#pragma unroll
      for (int e = 0; e < 4; ++e) S_g[(size_t)(q * 4 * R + 4 * rl + e) * P + j] = S[4 * q + e];
  }
}

template <int N, int Q, int COLS>
static cudaError_t launch_ssd_fixed(float* y, const float* xbc, const float* dtd, const pieh_ssd& s, const pieh_batch& b,
                                    cudaStream_t st) {
  constexpr int NT = N / (4 * Q) * COLS;
  constexpr size_t smem = (size_t)2 * kFixChunk * (2 * N + COLS + 2) * 4;
  static bool opted = false;
  if (smem > 48 * 1024 && !opted) {
    cudaFuncSetAttribute(ssd_scan_fixed_kernel<N, Q, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    opted = true;
  }
  return launch_k(ssd_scan_fixed_kernel<N, Q, COLS>, dim3((s.P + COLS - 1) / COLS, s.H, b.n_seq), dim3(NT), smem, st, y, xbc,
                  dtd, s, b);
}

static bool ssd_ok(const pieh_ssd* s) {
  return s && s->H > 0 && s->P > 0 && s->N > 0 && s->G > 0 && s->H % s->G == 0 && s->taps >= 1 && s->taps <= kSsdMaxTaps &&
         s->N <= 512 && s->xbc_off >= 0 && s->dt_off >= 0 && s->conv_w && s->dt_bias && s->A_log && s->state &&
         (s->taps == 1 || s->conv_state) && s->H <= 65535;
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_ssd_prepare(float* xbc, float* dtd, const float* proj, long long ld, const pieh_ssd* s,
                                const pieh_batch* b, void* stream) {
  if (!xbc || !dtd || !proj || !s || !b) return PIE_ENULL;
  if (!ssd_ok(s) || b->n_seq > 65535) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  count_launch(s->taps > 1 ? 2 : 1);
  launch_k(ssd_prepare_kernel, dim3(b->T), dim3(256), 0, st, xbc, dtd, proj, ld, *s, *b);
  if (s->taps > 1) {
    const int C = s->H * s->P + 2 * s->G * s->N;
    launch_k(ssd_advance_kernel, dim3((C + 127) / 128, b->n_seq), dim3(128), 0, st, proj, ld, *s, *b);
  }
  return status_of(cudaGetLastError());
}

extern "C" int pieh_ssd_scan(float* y, const float* xbc, const float* dtd, const pieh_ssd* s, const pieh_batch* b,
                             void* stream) {
  if (!y || !xbc || !dtd || !s || !b) return PIE_ENULL;
  if (!ssd_ok(s) || b->n_seq > 65535) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  const bool aligned = ((s->H * s->P) & 3) == 0 && (reinterpret_cast<uintptr_t>(xbc) & 15) == 0;
  static const bool generic_only = [] { const char* e = getenv("PIE_HYBRID_NO_FIXED_SCAN"); return e && e[0] == '1'; }();
  if (aligned && !generic_only && (s->N == 16 || s->N == 32 || s->N == 64 || s->N == 128)) {
    count_launch();
    cudaStream_t st = (cudaStream_t)stream;
    // measured at N = 128, P = 64, 32 heads, one 4096-row portion: 4 / 8 / 16 rows per lane 0.81 / 0.64 / 0.70 ms
    if (s->N == 128) return status_of(launch_ssd_fixed<128, 2, 16>(y, xbc, dtd, *s, *b, st));
    return status_of(s->N == 16 ? launch_ssd_fixed<16, 1, 32>(y, xbc, dtd, *s, *b, st)
                     : s->N == 32 ? launch_ssd_fixed<32, 1, 16>(y, xbc, dtd, *s, *b, st)
                     : s->N == 64 ? launch_ssd_fixed<64, 1, 16>(y, xbc, dtd, *s, *b, st)
                                  : launch_ssd_fixed<128, 1, 16>(y, xbc, dtd, *s, *b, st));
  }
  constexpr int RPT = 16;            // rows of a state column per lane
  int R = 1;
  while (R * RPT < s->N) R <<= 1;    // lanes per column, a power of two <= 32
  const int cols = kSsdThreads / R;
  const size_t smem = (size_t)2 * kSsdChunk * (2 * s->N + cols + 2) * 4;
  static bool opted = false;
  if (smem > 48 * 1024 && !opted) {
    cudaFuncSetAttribute(ssd_scan_kernel<RPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    opted = true;
  }
  count_launch();
  return status_of(launch_k(ssd_scan_kernel<RPT>, dim3((s->P + cols - 1) / cols, s->H, b->n_seq), dim3(kSsdThreads), smem,
                            (cudaStream_t)stream, y, xbc, dtd, *s, *b, R));
}
