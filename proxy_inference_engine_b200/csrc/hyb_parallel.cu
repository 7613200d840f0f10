// Pieces of parallel pre-norm blocks (one norm feeds the mixer and the feed-forward, both outputs join the residual together):
//   embed_scaled_kernel    x[t] = table[token] * scale
//   residual_norm_kernel   x[t] += y[t] + mixture of experts' rows (+ shared rows);  h[t] = rms_norm(x[t]) * w  -- the next
//                          block's norm in the pass that closes this block, so the residual is read once per block
//   canon_kernel           out_k[t] = h[t] + causal per-channel convolution of h (several tap sets over one h); rows before
//                          the step come from the sequence's state slot, rows before the sequence are zero
//   canon_state_kernel     afterwards: the last taps - 1 rows of h of every sequence become its state
//   mingru_*_kernel        S_t = (1 - z_t) S_(t-1) + z_t c_t per channel: one pass for short sequences, three passes over
//                          64-row tiles for long portions (a tile is a linear map of its incoming state)
//   latent_prepare_kernel  the two RMS norms of latent attention: query latent -> act tensor, key / value latent -> pages
//   rot_table_kernel       (cos, sin) of every row's rotation angles, formed once per step for all layers that share them
#include "hyb_common.cuh"

namespace pieh {

constexpr int kPageTokens = 64;

template <typename ET>
__global__ void embed_scaled_kernel(float* x, const ET* table, const int32_t* tokens, float scale, int W, int vocab) {
  pdl_sync();
  const int t = blockIdx.x;
  int id = tokens[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const ET* row = table + (size_t)id * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) x[(size_t)t * W + c] = elem<ET>::load(row + c) * scale;
}

__global__ void __launch_bounds__(256) residual_norm_kernel(float* x, const float* y, const pieh_mix_sum mix, float* h,
                                                            const float* norm_w, float eps, int W) {
  extern __shared__ float row[];
  __shared__ float red[33];
  pdl_sync();
  const int t = blockIdx.x;
  float ss = 0.f;
  float sg = 1.f;
  if (mix.parts && mix.shared && mix.shared_gate) sg = 1.f / (1.f + expf(-mix.shared_gate[(size_t)t * mix.gate_ld]));
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float add = y ? y[(size_t)t * W + c] : 0.f;
    if (mix.parts) {
      float v = 0.f;
      for (int k = 0; k < mix.top; ++k)   // choice order: the sum does not depend on how the slots were handed out
        v = fmaf(mix.part_w[(size_t)t * mix.top + k], mix.parts[(size_t)mix.part_row[(size_t)t * mix.top + k] * W + c], v);
      if (mix.shared) v = fmaf(sg, mix.shared[(size_t)t * W + c], v);
      add += v;
    }
    float v = x[(size_t)t * W + c];
    if (y || mix.parts) {
      v += add;
      x[(size_t)t * W + c] = v;
    }
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  if (!h || !norm_w) return;
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) h[(size_t)t * W + c] = row[c] * inv * norm_w[c];
}

constexpr int kMaxTaps = 8;

template <typename OT>
__global__ void __launch_bounds__(256) canon_kernel(const pieh_canon cn, const float* h, int W, const pieh_batch b) {
  pdl_sync();
  const int t = blockIdx.x;
  const int i = b.tok_seq[t], p = b.tok_pos[t], ctx = b.seq_ctx[i];
  const int taps = cn.taps;
  const float* hist = cn.state + (size_t)b.seq_slot[i] * (taps - 1) * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float past[kMaxTaps];   // past[j]: h of position p - taps + 1 + j; past[taps - 1] is this row
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
      if (j < taps) {
        const int pp = p - taps + 1 + j;
        float v = 0.f;
        if (pp >= ctx) v = h[(size_t)(t - (p - pp)) * W + c];                          // a row of this step
        else if (pp >= 0) v = hist[(size_t)(pp - ctx + taps - 1) * W + c];             // a row of an earlier step
        past[j] = v;
      }
    }
    const float cur = past[taps - 1];
    for (int k = 0; k < cn.n_out; ++k) {
      const float* w = cn.w[k] + (size_t)c * taps;
      float acc = cur;
#pragma unroll
      for (int j = 0; j < kMaxTaps; ++j)
        if (j < taps) acc = fmaf(w[j], past[j], acc);
      elem<OT>::store(reinterpret_cast<OT*>(cn.out[k]) + (size_t)t * W + c, acc);
    }
  }
}

__device__ __forceinline__ void store4(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), c = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&c));
}

// W a multiple of 4: a thread owns 4 neighbouring channels and walks kCanonRows consecutive rows of the step with the last
// taps - 1 rows of h in registers, so h is read once (plus the warm-up rows of a tile); its taps stay in registers too.
// Where a row starts another sequence (or the tile) the window is fetched anew: this step's rows, the state slot, or zeros.
constexpr int kCanonRows = 16;
template <typename OT, int MAXT, int NOUT>   // array sizes: taps <= MAXT, tap sets <= NOUT (registers, hence occupancy)
__global__ void __launch_bounds__(128) canon_rows_kernel(const pieh_canon cn, const float* h, int W, const pieh_batch b) {
  pdl_sync();
  const int c = (blockIdx.x * 128 + threadIdx.x) * 4;
  if (c >= W) return;
  const int t0 = blockIdx.y * kCanonRows, t1 = min(b.T, t0 + kCanonRows);
  const int taps = cn.taps;
  float wt[NOUT][MAXT][4];   // [tap set][tap][channel]
#pragma unroll
  for (int k = 0; k < NOUT; ++k)
    if (k < cn.n_out)
#pragma unroll
      for (int j = 0; j < MAXT; ++j)
        if (j < taps)
#pragma unroll
          for (int e = 0; e < 4; ++e) wt[k][j][e] = cn.w[k][(size_t)(c + e) * taps + j];
  float past[MAXT][4];    // past[j]: h of the row's position - (taps - 1) + j, j < taps - 1
  int prev = -1;
  for (int t = t0; t < t1; ++t) {
    const int i = b.tok_seq[t];
    if (i != prev) {
      const int p = b.tok_pos[t], ctx = b.seq_ctx[i];
      const float* hist = cn.state + (size_t)b.seq_slot[i] * (taps - 1) * W;
#pragma unroll
      for (int j = 0; j < MAXT - 1; ++j) {
        if (j < taps - 1) {
          const int pp = p - taps + 1 + j;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (pp >= ctx) v = *reinterpret_cast<const float4*>(h + (size_t)(t - (p - pp)) * W + c);
          else if (pp >= 0) v = *reinterpret_cast<const float4*>(hist + (size_t)(pp - ctx + taps - 1) * W + c);
          past[j][0] = v.x; past[j][1] = v.y; past[j][2] = v.z; past[j][3] = v.w;
        }
      }
      prev = i;
    }
    const float4 cv = *reinterpret_cast<const float4*>(h + (size_t)t * W + c);
    const float cur[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
    for (int k = 0; k < NOUT; ++k) {
      if (k < cn.n_out) {
        float acc[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = cur[e];
#pragma unroll
        for (int j = 0; j < MAXT; ++j) {
          if (j < taps - 1) {
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fmaf(wt[k][j][e], past[j][e], acc[e]);
          } else if (j == taps - 1) {
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fmaf(wt[k][j][e], cur[e], acc[e]);
          }
        }
        store4(reinterpret_cast<OT*>(cn.out[k]) + (size_t)t * W + c, acc);
      }
    }
#pragma unroll
    for (int j = 0; j < MAXT - 1; ++j) {
      if (j < taps - 1) {
#pragma unroll
        for (int e = 0; e < 4; ++e) past[j][e] = j + 1 < taps - 1 ? past[j + 1][e] : cur[e];
      }
    }
  }
}

// one CTA row per sequence: state[s] <- h of position ctx + n - (taps - 1) + s
__global__ void __launch_bounds__(256) canon_state_kernel(const pieh_canon cn, const float* h, int W, const pieh_batch b) {
  pdl_sync();
  const int i = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= W) return;
  const int start = b.seq_start[i], n = b.seq_len[i], ctx = b.seq_ctx[i], taps = cn.taps;
  float* hist = cn.state + (size_t)b.seq_slot[i] * (taps - 1) * W;
  float keep[kMaxTaps];
#pragma unroll
  for (int s = 0; s < kMaxTaps - 1; ++s) {
    if (s < taps - 1) {
      const int pp = ctx + n - (taps - 1) + s;
      float v = 0.f;
      if (pp >= ctx) v = h[(size_t)(start + pp - ctx) * W + c];
      else if (pp >= 0) v = hist[(size_t)(pp - ctx + taps - 1) * W + c];
      keep[s] = v;
    }
  }
#pragma unroll
  for (int s = 0; s < kMaxTaps - 1; ++s)
    if (s < taps - 1) hist[(size_t)s * W + c] = keep[s];
}

// The gates of row r, from the fused projection: keep = 1 - z, add = z * candidate
__device__ __forceinline__ void mingru_gates(const float* row, int width, float& keep, float& add) {
  const float z = 1.f / (1.f + expf(-row[0]));
  const float u = row[width];
  const float cand = u >= 0.f ? u + 0.5f : 1.f / (1.f + expf(-u));
  keep = 1.f - z;
  add = z * cand;
}

// Short sequences (every sequence's rows fit one 64-row tile: decoding, small portions): one pass, a thread per channel.
template <typename OT>
__global__ void __launch_bounds__(64) mingru_scan_kernel(OT* out, const float* proj, long long ld, int width, float* state,
                                                         const pieh_batch b) {
  pdl_sync();
  const int i = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int start = b.seq_start[i], n = b.seq_len[i];
  float* sp = state + (size_t)b.seq_slot[i] * width + c;
  float S = b.seq_ctx[i] > 0 ? *sp : 0.f;
  constexpr int RUN = 8;
  for (int r0 = 0; r0 < n; r0 += RUN) {
    float keep[RUN], add[RUN], gate[RUN];
#pragma unroll
    for (int r = 0; r < RUN; ++r) {
      if (r0 + r < n) {
        const float* row = proj + (size_t)(start + r0 + r) * ld + c;
        mingru_gates(row, width, keep[r], add[r]);
        gate[r] = silu_f(row[2 * (size_t)width]);
      }
    }
#pragma unroll
    for (int r = 0; r < RUN; ++r) {
      if (r0 + r < n) {
        S = fmaf(keep[r], S, add[r]);
        elem<OT>::store(out + (size_t)(start + r0 + r) * width + c, S * gate[r]);
      }
    }
  }
  *sp = S;
}

// Long portions: the recurrence S <- keep S + add is linear in S, so a 64-row tile acts on its incoming state as
// S_out = A S_in + B with A = prod keep and B = the tile's own scan from zero.
//   pass 1 (a CTA per tile and 128 channels): A and B of every tile
//   pass 2 (a thread per sequence and channel): walks the sequence's tiles in order -> the state each tile starts from,
//           and the sequence's new state
//   pass 3 (as pass 1): the scan again from the true incoming state, times silu(gate), to the output
// scratch: [3, n_tiles, width] floats (A, B, incoming state).
constexpr int kScanRun = 8;
__global__ void __launch_bounds__(128) mingru_tile_kernel(const float* proj, long long ld, int width, float* scratch,
                                                          const pieh_batch b) {
  pdl_sync();
  const int tile = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int i = b.tile_seq[tile], row0 = b.tile_row[tile];
  const int n = min(64, b.seq_start[i] + b.seq_len[i] - row0);
  float A = 1.f, B = 0.f;
  for (int r0 = 0; r0 < n; r0 += kScanRun) {
    float keep[kScanRun], add[kScanRun];
#pragma unroll
    for (int r = 0; r < kScanRun; ++r)
      if (r0 + r < n) mingru_gates(proj + (size_t)(row0 + r0 + r) * ld + c, width, keep[r], add[r]);
#pragma unroll
    for (int r = 0; r < kScanRun; ++r)
      if (r0 + r < n) { A *= keep[r]; B = fmaf(keep[r], B, add[r]); }
  }
  scratch[(size_t)tile * width + c] = A;
  scratch[((size_t)b.n_tiles + tile) * width + c] = B;
}

__global__ void __launch_bounds__(128) mingru_carry_kernel(int width, float* scratch, float* state, const pieh_batch b) {
  pdl_sync();
  const int i = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  int tile = 0;   // the tile list holds every sequence's tiles in sequence order
  for (int j = 0; j < i; ++j) tile += (b.seq_len[j] + 63) / 64;
  const int nt = (b.seq_len[i] + 63) / 64;
  float* sp = state + (size_t)b.seq_slot[i] * width + c;
  float S = b.seq_ctx[i] > 0 ? *sp : 0.f;
  for (int k0 = 0; k0 < nt; k0 += kScanRun, tile += kScanRun) {   // the loads of a run do not wait for the chain
    float A[kScanRun], B[kScanRun];
#pragma unroll
    for (int k = 0; k < kScanRun; ++k) {
      if (k0 + k < nt) {
        A[k] = scratch[(size_t)(tile + k) * width + c];
        B[k] = scratch[((size_t)b.n_tiles + tile + k) * width + c];
      }
    }
#pragma unroll
    for (int k = 0; k < kScanRun; ++k) {
      if (k0 + k < nt) {
        scratch[((size_t)2 * b.n_tiles + tile + k) * width + c] = S;
        S = fmaf(A[k], S, B[k]);
      }
    }
  }
  *sp = S;
}

template <typename OT>
__global__ void __launch_bounds__(128) mingru_apply_kernel(OT* out, const float* proj, long long ld, int width,
                                                           const float* scratch, const pieh_batch b) {
  pdl_sync();
  const int tile = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int i = b.tile_seq[tile], row0 = b.tile_row[tile];
  const int n = min(64, b.seq_start[i] + b.seq_len[i] - row0);
  float S = scratch[((size_t)2 * b.n_tiles + tile) * width + c];
  for (int r0 = 0; r0 < n; r0 += kScanRun) {
    float keep[kScanRun], add[kScanRun], gate[kScanRun];
#pragma unroll
    for (int r = 0; r < kScanRun; ++r) {
      if (r0 + r < n) {
        const float* row = proj + (size_t)(row0 + r0 + r) * ld + c;
        mingru_gates(row, width, keep[r], add[r]);
        gate[r] = silu_f(row[2 * (size_t)width]);
      }
    }
#pragma unroll
    for (int r = 0; r < kScanRun; ++r) {
      if (r0 + r < n) {
        S = fmaf(keep[r], S, add[r]);
        elem<OT>::store(out + (size_t)(row0 + r0 + r) * width + c, S * gate[r]);
      }
    }
  }
}

template <typename OT, typename KT>
__global__ void __launch_bounds__(256) latent_prepare_kernel(OT* cq_out, const float* proj, long long ld, int q_rank,
                                                             long long kv_off, int kv_rank, const float* q_norm,
                                                             const float* kv_norm, float eps, KT* pages, const pieh_batch b) {
  __shared__ float red[33];
  pdl_sync();
  const int t = blockIdx.x;
  const int i = b.tok_seq[t], p = b.tok_pos[t];
  const float* row = proj + (size_t)t * ld;
  float ss = 0.f;
  for (int c = threadIdx.x; c < q_rank; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
  const float iq = 1.f / sqrtf(block_sum(ss, red) / (float)q_rank + eps);
  ss = 0.f;
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) ss = fmaf(row[kv_off + c], row[kv_off + c], ss);
  const float ik = 1.f / sqrtf(block_sum(ss, red) / (float)kv_rank + eps);
  for (int c = threadIdx.x; c < q_rank; c += blockDim.x) elem<OT>::store(cq_out + (size_t)t * q_rank + c, row[c] * iq * q_norm[c]);
  const size_t slot = (size_t)b.block_table[(size_t)i * b.bt_stride + p / kPageTokens] * kPageTokens + p % kPageTokens;
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x)
    elem<KT>::store(pages + slot * kv_rank + c, row[kv_off + c] * ik * kv_norm[c]);
}

__global__ void rot_table_kernel(float* cs, const int32_t* positions, const double* freqs, int half, long long n) {
  pdl_sync();
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const long long t = e / half;
  const int i = (int)(e - t * half);
  double s, c;
  sincos((double)positions[t] * freqs[i], &s, &c);
  cs[2 * e] = (float)c;
  cs[2 * e + 1] = (float)s;
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_embed_scaled(float* x, const void* table, int table_dtype, const int32_t* tokens, float scale, int T,
                                 int W, int vocab, void* stream) {
  if (!x || !table || !tokens) return PIE_ENULL;
  if (T < 0 || W < 1 || vocab < 1) return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  count_launch();
  PIEH_DISPATCH_DTYPE(table_dtype, ET, launch_k(embed_scaled_kernel<ET>, dim3(T), dim3(256), 0, (cudaStream_t)stream, x,
                                                (const ET*)table, tokens, scale, W, vocab));
  return status_of(cudaGetLastError());
}

extern "C" int pieh_residual_norm(float* x, const float* y, const pieh_mix_sum* mix, float* h, const float* norm_w,
                                  float eps, int T, int W, void* stream) {
  if (!x) return PIE_ENULL;
  if (mix && mix->parts && (!mix->part_row || !mix->part_w || mix->top < 1)) return PIE_ENULL;
  if (T < 0 || W < 1 || (size_t)W * 4 > 200 * 1024) return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  pieh_mix_sum m = {};
  if (mix && mix->parts) m = *mix;
  const size_t smem = (size_t)W * 4;
  if (smem > 48 * 1024) cudaFuncSetAttribute(residual_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  count_launch();
  launch_k(residual_norm_kernel, dim3(T), dim3(256), smem, (cudaStream_t)stream, x, y, m, h, norm_w, eps, W);
  return status_of(cudaGetLastError());
}

extern "C" int pieh_canon_conv(const pieh_canon* c, int out_dtype, const float* h, int W, const pieh_batch* b, void* stream) {
  if (!c || !h || !b) return PIE_ENULL;
  if (c->taps < 1 || c->taps > kMaxTaps || c->n_out < 1 || c->n_out > 4 || W < 1) return PIE_EINVAL_SHAPE;
  for (int k = 0; k < c->n_out; ++k)
    if (!c->w[k] || !c->out[k]) return PIE_ENULL;
  if (c->taps > 1 && !c->state) return PIE_ENULL;
  if (b->T == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  count_launch();
  bool aligned = W % 4 == 0 && (reinterpret_cast<uintptr_t>(h) & 15) == 0 && (!c->state || (reinterpret_cast<uintptr_t>(c->state) & 15) == 0);
  for (int k = 0; k < c->n_out; ++k) aligned = aligned && (reinterpret_cast<uintptr_t>(c->out[k]) & 15) == 0;
  if (aligned) {
    const dim3 grid((W + 511) / 512, (b->T + kCanonRows - 1) / kCanonRows);
#define PIEH_CANON(MAXT, NOUT) PIEH_DISPATCH_DTYPE(out_dtype, OT, launch_k(canon_rows_kernel<OT, MAXT, NOUT>, grid, dim3(128), 0, st, *c, h, W, *b))
    if (c->taps <= 4 && c->n_out <= 2) PIEH_CANON(4, 2);
    else if (c->taps <= 4) PIEH_CANON(4, 4);
    else if (c->n_out <= 2) PIEH_CANON(8, 2);
    else PIEH_CANON(8, 4);
#undef PIEH_CANON
  } else
    PIEH_DISPATCH_DTYPE(out_dtype, OT, launch_k(canon_kernel<OT>, dim3(b->T), dim3(256), 0, st, *c, h, W, *b));
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && c->taps > 1) {
    count_launch();
    e = launch_k(canon_state_kernel, dim3((W + 255) / 256, b->n_seq), dim3(256), 0, st, *c, h, W, *b);
  }
  return status_of(e);
}

extern "C" int pieh_mingru_scan(void* out, int out_dtype, const float* proj, long long ld, int width, float* state,
                                float* scratch, const pieh_batch* b, void* stream) {
  if (!out || !proj || !state || !b) return PIE_ENULL;
  if (width < 1 || ld < 3LL * width) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool tiled = scratch && b->n_tiles > b->n_seq && b->tile_seq && b->tile_row;   // some sequence spans several tiles
  if (!tiled) {
    count_launch();
    PIEH_DISPATCH_DTYPE(out_dtype, OT, launch_k(mingru_scan_kernel<OT>, dim3((width + 63) / 64, b->n_seq), dim3(64), 0, st,
                                                (OT*)out, proj, ld, width, state, *b));
    return status_of(cudaGetLastError());
  }
  count_launch(3);
  const dim3 grid((width + 127) / 128, b->n_tiles);
  cudaError_t e = launch_k(mingru_tile_kernel, grid, dim3(128), 0, st, proj, ld, width, scratch, *b);
  if (e == cudaSuccess)
    e = launch_k(mingru_carry_kernel, dim3((width + 127) / 128, b->n_seq), dim3(128), 0, st, width, scratch, state, *b);
  if (e == cudaSuccess) {
    PIEH_DISPATCH_DTYPE(out_dtype, OT, launch_k(mingru_apply_kernel<OT>, grid, dim3(128), 0, st, (OT*)out, proj, ld, width,
                                                (const float*)scratch, *b));
    e = cudaGetLastError();
  }
  return status_of(e);
}

extern "C" int pieh_latent_prepare(void* cq_out, int out_dtype, const float* proj, long long ld, int q_rank, long long kv_off,
                                   int kv_rank, const float* q_norm, const float* kv_norm, float eps, void* pages,
                                   int kv_dtype, const pieh_batch* b, void* stream) {
  if (!cq_out || !proj || !q_norm || !kv_norm || !pages || !b) return PIE_ENULL;
  if (q_rank < 1 || kv_rank < 1 || kv_off < 0) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  count_launch();
  PIEH_DISPATCH_DTYPE(out_dtype, OT, PIEH_DISPATCH_DTYPE(kv_dtype, KT,
      launch_k(latent_prepare_kernel<OT, KT>, dim3(b->T), dim3(256), 0, (cudaStream_t)stream, (OT*)cq_out, proj, ld, q_rank,
               kv_off, kv_rank, q_norm, kv_norm, eps, (KT*)pages, *b)));
  return status_of(cudaGetLastError());
}

extern "C" int pieh_rot_table(float* cs, const int32_t* positions, const double* freqs, int T, int half, void* stream) {
  if (!cs || !positions || !freqs) return PIE_ENULL;
  if (T < 0 || half < 1) return PIE_EINVAL_SHAPE;
  if (T == 0) return PIE_OK;
  const long long n = (long long)T * half;
  count_launch();
  launch_k(rot_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, cs, positions, freqs, half, n);
  return status_of(cudaGetLastError());
}
