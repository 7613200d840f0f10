// Attention with a per-head linear distance bias, a softmax sink and a sigmoid output gate over 64-token pages, ragged steps.
//   s_ij = q_i . k_j * scale - slope_h (i - j),  j <= i (and i - j < window if one is set)
//   p_ij = exp(s_ij) / (sink + sum_j exp(s_ij))          sink = 1: a term of score 0 that carries no value, so a query
//                                                        that matches nothing returns (almost) nothing
//   out_i = sum_j p_ij v_j * sigmoid(gate_i)
// Optional: a LEARNED sink logit per head in place of the score-0 sink, one gate logit per head in place of one per
// feature, a rotation of the leading features of every query / key head ("rotate half" pairing) from a per-step (cos, sin)
// table, and values blended with another layer's values of the same token before they are cached.
// bias_prepare_kernel   per token: ONE rms norm over all heads' query features (and one over all key features) with
//                       per-feature weights, the query temperature 1 + c ln(floor((p + 1) / every) + 1), then the normed
//                       keys go to the key pages and the values -- here usually the PROJECTED keys themselves, v_off ==
//                       k_off -- to the value pages at the token's position
// bias_run_kernel       one CTA per (token, query head): 8 warps take 32-key blocks in turn with an online softmax each,
//                       merged through shared memory together with the sink; serves decoding and every fp32 step.
//                       When a step has few (token, head) pairs -- decoding -- a thread-block CLUSTER of 2 / 4 / 8 CTAs
//                       shares one pair: each CTA takes a contiguous slice of the keys and the first CTA of the cluster
//                       reads the others' partial softmax out of their shared memory (distributed shared memory), so a
//                       long context is spread over the whole GPU without a workspace or a second launch
// bias_tile_kernel      prompt portions over bf16 pages: 64-row query tiles on mma.sync (below)
// A step's keys are appended before its queries run, so a prompt portion sees itself through the same pages as its past.
#include <cooperative_groups.h>

#include "hyb_common.cuh"

namespace pieh {

namespace cg = cooperative_groups;
constexpr int kPage = 64;

template <typename KT>
__global__ void __launch_bounds__(256) bias_prepare_kernel(float* q_out, const float* proj, long long ld,
                                                           const pieh_bias_attn a, const pieh_batch b) {
  __shared__ float red[33];
  pdl_sync();
  const int t = blockIdx.x;
  const int i = b.tok_seq[t], p = b.tok_pos[t];
  const int nq = a.H * a.d, nk = a.G * a.d, nv = a.G * a.dv;
  const float* row = proj + (size_t)t * ld;
  float iq = 1.f, ik = 1.f;
  if (a.q_norm) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
    iq = 1.f / sqrtf(block_sum(ss, red) / (float)nq + a.eps);
  }
  if (a.k_norm) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < nk; c += blockDim.x) ss = fmaf(row[a.k_off + c], row[a.k_off + c], ss);
    ik = 1.f / sqrtf(block_sum(ss, red) / (float)nk + a.eps);
  }
  if (a.temp_every > 0.0) iq *= 1.f + a.temp_coef * logf((float)floor((double)(p + 1) / a.temp_every) + 1.f);
  const size_t slot = (size_t)b.block_table[(size_t)i * b.bt_stride + p / kPage] * kPage + p % kPage;
  KT* kp = reinterpret_cast<KT*>(a.k_pages) + slot * nk;
  KT* vp = reinterpret_cast<KT*>(a.v_pages) + slot * nv;
  // feature c of a projection after its norm and, for the leading rot_dims features of a head, the rotation that pairs
  // feature f with f + rot_dims / 2
  const int half = a.rot_dims >> 1;
  const float* cs = a.rot_cs ? a.rot_cs + (size_t)t * half * 2 : nullptr;
  auto feat = [&](const float* x, const float* nw, float inv, int c) {
    const float v = x[c] * inv * (nw ? nw[c] : 1.f);
    const int f = c % a.d;
    if (!cs || f >= a.rot_dims) return v;
    const bool lo = f < half;
    const int o = lo ? c + half : c - half;
    const float u = x[o] * inv * (nw ? nw[o] : 1.f);
    const float co = cs[2 * (lo ? f : f - half)], si = cs[2 * (lo ? f : f - half) + 1];
    return lo ? v * co - u * si : v * co + u * si;
  };
  for (int c = threadIdx.x; c < nq; c += blockDim.x) q_out[(size_t)t * nq + c] = feat(row, a.q_norm, iq, c);
  for (int c = threadIdx.x; c < nk; c += blockDim.x) elem<KT>::store(kp + c, feat(row + a.k_off, a.k_norm, ik, c));
  const float lam = a.v_mix ? *a.v_mix : 0.f;
  for (int c = threadIdx.x; c < nv; c += blockDim.x) {
    float v = row[a.v_off + c];
    if (a.v_mix) v = (1.f - lam) * v + lam * a.v_keep[(size_t)t * nv + c];
    else if (a.v_keep) a.v_keep[(size_t)t * nv + c] = v;
    elem<KT>::store(vp + c, v);
  }
}

constexpr int kRunWarps = 8;

template <typename T> struct ld8;   // 8 consecutive cache elements as floats
template <> struct ld8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct ld8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
};

template <typename KT, typename OT, int NV, bool CLUSTER>
__global__ void __launch_bounds__(kRunWarps * 32) bias_run_kernel(OT* out, const float* q, const float* proj, long long ld,
                                                                  const pieh_bias_attn a, const pieh_batch b, int cs) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NW = kRunWarps, NTH = kRunWarps * 32;
  pdl_sync();
  const int pair = blockIdx.x / cs, rank = blockIdx.x - pair * cs;   // cs CTAs (one cluster) per (token, head)
  const int t = pair / a.H, h = pair - t * a.H;
  const int g = h / (a.H / a.G);
  const int i = b.tok_seq[t], p = b.tok_pos[t];
  const int d = a.d, dv = a.dv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = sm;                       // [d]
  float* mg = qs + d;                   // [warps][dv + 2]: acc, m, l
  float* part = mg + NW * (dv + 2);     // [dv + 2]: this CTA's merged partial softmax
  for (int c = threadIdx.x; c < d; c += NTH) qs[c] = q[((size_t)t * a.H + h) * d + c];
  __syncthreads();
  const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
  // this CTA's slice of the keys lo .. p: whole 32-key blocks, in order of rank
  const int chunk = ((p - lo + cs) / cs + 31) / 32 * 32;
  const int my_lo = lo + rank * chunk, my_hi = min(p, my_lo + chunk - 1);
  const float slope = a.slopes ? a.slopes[h] : 0.f;
  // sigmoid weights: no maximum, no denominator -- every partial result is a plain sum (m stays 0, so every merge factor is 1)
  const bool sgm = a.sigmoid != 0;
  const float sbias = sgm && a.score_bias ? a.score_bias[h] : 0.f;
  const int32_t* table = b.block_table + (size_t)i * b.bt_stride;
  const KT* kpool = reinterpret_cast<const KT*>(a.k_pages);
  const KT* vpool = reinterpret_cast<const KT*>(a.v_pages);
  const bool vec = (d & 7) == 0;
  float m = sgm ? 0.f : -1e30f, l = 0.f, acc[NV];
#pragma unroll
  for (int x = 0; x < NV; ++x) acc[x] = 0.f;
  for (int base = my_lo + warp * 32; base <= my_hi; base += NW * 32) {
    const int j = base + lane;
    const bool ok = j <= my_hi;
    long long slot = 0;
    float s = -1e30f;
    if (ok) {
      slot = (long long)table[j / kPage] * kPage + j % kPage;
      const KT* kr = kpool + ((size_t)slot * a.G + g) * d;
      float dot = 0.f;
      if (vec) {
#pragma unroll 4
        for (int c = 0; c < d; c += 8) {
          float kk[8];
          ld8<KT>::load(kr + c, kk);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(qs[c + e], kk[e], dot);
        }
      } else {
        for (int c = 0; c < d; ++c) dot = fmaf(qs[c], elem<KT>::load(kr + c), dot);
      }
      s = dot * a.scale - slope * (float)(p - j);
    }
    float pj;
    if (sgm) {
      pj = ok ? 1.f / (1.f + expf(-(s + sbias))) : 0.f;
    } else {
      const float n = fmaxf(m, warp_max(s));
      const float cf = expf(m - n);
      pj = ok ? expf(s - n) : 0.f;
      l = l * cf + warp_sum(pj);
      m = n;
#pragma unroll
      for (int x = 0; x < NV; ++x) acc[x] *= cf;
    }
#pragma unroll 1
    for (int k0 = 0; k0 < 32; k0 += 4) {
      if (base + k0 > my_hi) break;
      float w[4], vv[4][NV];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        w[u] = __shfl_sync(0xffffffffu, pj, k0 + u);
        const long long sl = __shfl_sync(0xffffffffu, slot, k0 + u);
        const KT* vr = vpool + ((size_t)sl * a.G + g) * dv;
#pragma unroll
        for (int x = 0; x < NV; ++x) {
          const int c = lane + 32 * x;
          vv[u][x] = c < dv ? elem<KT>::load(vr + c) : 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int x = 0; x < NV; ++x) acc[x] = fmaf(w[u], vv[u][x], acc[x]);
    }
  }
  float* mine = mg + (size_t)warp * (dv + 2);
#pragma unroll
  for (int x = 0; x < NV; ++x) {
    const int c = lane + 32 * x;
    if (c < dv) mine[c] = acc[x];
  }
  if (lane == 0) { mine[dv] = m; mine[dv + 1] = l; }
  __syncthreads();
  {                            // the warps of this CTA -> one partial softmax
    float M = sgm ? 0.f : -1e30f, f[NW], L = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, mg[(size_t)w * (dv + 2) + dv]);
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      f[w] = expf(mg[(size_t)w * (dv + 2) + dv] - M);
      L = fmaf(mg[(size_t)w * (dv + 2) + dv + 1], f[w], L);
    }
    for (int c = threadIdx.x; c < dv; c += NTH) {
      float A = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) A = fmaf(mg[(size_t)w * (dv + 2) + c], f[w], A);
      part[c] = A;
    }
    if (threadIdx.x == 0) { part[dv] = M; part[dv + 1] = L; }
  }
  if (CLUSTER) cg::this_cluster().sync(); else __syncthreads();
  if (rank == 0) {   // the CTAs of the cluster and the sink -> the output
    // the sink is one more partial softmax: maximum = its logit (0 for the fixed sink), sum 1, no values
    const bool has_sink = !sgm && (a.sinks != nullptr || a.sink != 0);
    const float sk = a.sinks ? a.sinks[h] : 0.f;
    float M = sgm ? 0.f : has_sink ? sk : -1e30f;
    float L = 0.f;
    const float* gate = a.g_off >= 0 ? proj + (size_t)t * ld + a.g_off + (a.gate_heads ? (size_t)h : (size_t)h * dv) : nullptr;
    if (CLUSTER) {
      cg::cluster_group cl = cg::this_cluster();
      for (int r = 0; r < cs; ++r) M = fmaxf(M, cl.map_shared_rank(part, r)[dv]);
      for (int r = 0; r < cs; ++r) {
        const float* src = cl.map_shared_rank(part, r);
        L = fmaf(src[dv + 1], expf(src[dv] - M), L);
      }
      if (has_sink) L += expf(sk - M);
      for (int c = threadIdx.x; c < dv; c += NTH) {
        float A = 0.f;
        for (int r = 0; r < cs; ++r) {
          const float* src = cl.map_shared_rank(part, r);
          A = fmaf(src[c], expf(src[dv] - M), A);
        }
        float o = sgm ? A : A / L;
        if (gate) o *= 1.f / (1.f + expf(-gate[a.gate_heads ? 0 : c]));
        elem<OT>::store(out + ((size_t)t * a.H + h) * dv + c, o);
      }
    } else {
      M = fmaxf(M, part[dv]);
      const float f = expf(part[dv] - M);
      L = part[dv + 1] * f;
      if (has_sink) L += expf(sk - M);
      for (int c = threadIdx.x; c < dv; c += NTH) {
        float o = sgm ? part[c] : part[c] * f / L;
        if (gate) o *= 1.f / (1.f + expf(-gate[a.gate_heads ? 0 : c]));
        elem<OT>::store(out + ((size_t)t * a.H + h) * dv + c, o);
      }
    }
  }
  if (CLUSTER) cg::this_cluster().sync();   // nobody's shared memory goes away while the first CTA still reads it
}

// ---- prompt portions on the tensor cores ---------------------------------------------------------------------------
// A CTA of 4 warps owns one 64-row query tile (consecutive positions of ONE sequence) of one query head; key tiles are
// whole pages (64 keys) from the first page the window reaches to the page of the tile's last row, double-buffered in
// XOR-swizzled shared memory by cp.async.  S = Q K^T on mma.sync.m16n8k16 (bf16 in, fp32 out); scale, distance bias,
// causal and window mask, online softmax in fp32 (exp2 domain) whose running maximum starts at the sink's score 0, P
// rounded to bf16, O += P V.  The end adds the sink to the denominator, applies the output gate and stores bf16.
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
template <int ROWB>   // bytes of a tile row (>= 128); 16-byte chunk c of row r sits at chunk c ^ (r & 7)
__device__ __forceinline__ uint32_t tile_off(int r, int c) { return (uint32_t)(r * ROWB + ((c ^ (r & 7)) << 4)); }

template <int D, int DV>
__global__ void __launch_bounds__(128) bias_tile_kernel(__nv_bfloat16* out, const float* q, const float* proj, long long ld,
                                                        const pieh_bias_attn a, const pieh_batch b) {
  constexpr int KC = D / 16, NT = 8, DT = DV / 8;
  constexpr int KROWB = D * 2, VROWB = DV * 2;
  constexpr int KTILE = 64 * KROWB, VTILE = 64 * VROWB;
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_sync();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int tile = blockIdx.x, h = blockIdx.y;
  const int i = b.tile_seq[tile], row0 = b.tile_row[tile];
  const int nrows = min(64, b.seq_start[i] + b.seq_len[i] - row0);
  const int pos0 = b.tok_pos[row0];
  const int kvh = h / (a.H / a.G);
  const int last_key = pos0 + nrows - 1;
  const int first_key = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const int j_lo = first_key / kPage, j_hi = last_key / kPage;
  const int32_t* table = b.block_table + (size_t)i * b.bt_stride;
  const __nv_bfloat16* kpool = reinterpret_cast<const __nv_bfloat16*>(a.k_pages);
  const __nv_bfloat16* vpool = reinterpret_cast<const __nv_bfloat16*>(a.v_pages);
  const uint32_t sK = (uint32_t)__cvta_generic_to_shared(smem), sV = sK + 2 * KTILE;

  auto issue = [&](int j) {
    const size_t page = (size_t)table[j] * kPage;
    const uint32_t dk = sK + ((j - j_lo) & 1) * KTILE, dvv = sV + ((j - j_lo) & 1) * VTILE;
    constexpr int CK = KROWB / 16, CV = VROWB / 16;
    for (int e = tid; e < 64 * CK; e += 128) {
      const int r = e / CK, c = e - r * CK;
      cp16(dk + tile_off<KROWB>(r, c), kpool + ((page + r) * a.G + kvh) * D + c * 8);
    }
    for (int e = tid; e < 64 * CV; e += 128) {
      const int r = e / CV, c = e - r * CV;
      cp16(dvv + tile_off<VROWB>(r, c), vpool + ((page + r) * a.G + kvh) * DV + c * 8);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  issue(j_lo);

  // Q fragments: rows 16 warp + g and + 8 of the tile (rows past the tile's end repeat its last row)
  const int r0 = warp * 16 + g, r1 = r0 + 8;
  uint32_t qf[KC][4];
  {
    const float* q0 = q + ((size_t)(row0 + min(r0, nrows - 1)) * a.H + h) * D;
    const float* q1 = q + ((size_t)(row0 + min(r1, nrows - 1)) * a.H + h) * D;
#pragma unroll
    for (int kc = 0; kc < KC; ++kc) {
      const float2 x0 = *reinterpret_cast<const float2*>(q0 + kc * 16 + 2 * t4);
      const float2 x1 = *reinterpret_cast<const float2*>(q1 + kc * 16 + 2 * t4);
      const float2 x2 = *reinterpret_cast<const float2*>(q0 + kc * 16 + 8 + 2 * t4);
      const float2 x3 = *reinterpret_cast<const float2*>(q1 + kc * 16 + 8 + 2 * t4);
      qf[kc][0] = pack2(x0.x, x0.y); qf[kc][1] = pack2(x1.x, x1.y);
      qf[kc][2] = pack2(x2.x, x2.y); qf[kc][3] = pack2(x3.x, x3.y);
    }
  }
  float o[DT][4];
#pragma unroll
  for (int x = 0; x < DT; ++x) o[x][0] = o[x][1] = o[x][2] = o[x][3] = 0.f;
  constexpr float kLog2e = 1.4426950408889634f;
  const bool sgm = a.sigmoid != 0;                          // sigmoid weights: no running maximum, no denominator
  const float sb2 = sgm && a.score_bias ? a.score_bias[h] * kLog2e : 0.f;
  const bool has_sink = !sgm && (a.sinks != nullptr || a.sink != 0);
  const float sk2 = a.sinks ? a.sinks[h] * kLog2e : 0.f;   // the sink's logit in the exp2 domain
  const float m_init = has_sink ? sk2 : -INFINITY;
  float mrun[2] = {m_init, m_init}, lrun[2] = {0.f, 0.f};
  const int p0 = pos0 + min(r0, nrows - 1), p1 = pos0 + min(r1, nrows - 1);   // positions of this thread's two rows
  const int w0 = a.window > 0 ? p0 - a.window + 1 : 0, w1 = a.window > 0 ? p1 - a.window + 1 : 0;
  const float slope = a.slopes ? a.slopes[h] : 0.f;

  for (int j = j_lo; j <= j_hi; ++j) {
    if (j < j_hi) { issue(j + 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const uint32_t tk = sK + ((j - j_lo) & 1) * KTILE, tv = sV + ((j - j_lo) & 1) * VTILE;
    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
      for (int kc = 0; kc < KC; kc += 2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(tk + tile_off<KROWB>(n * 8 + (lane & 7), kc * 2 + (lane >> 3)), b0, b1, b2, b3);
        mma_16816(s[n], qf[kc][0], qf[kc][1], qf[kc][2], qf[kc][3], b0, b1);
        mma_16816(s[n], qf[kc + 1][0], qf[kc + 1][1], qf[kc + 1][2], qf[kc + 1][3], b2, b3);
      }
    }
    const int key0 = j * kPage + 2 * t4;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const int k = key0 + n * 8;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = k + (e & 1), pr = e < 2 ? p0 : p1, wl = e < 2 ? w0 : w1;
        const float v = s[n][e] * a.scale - slope * (float)(pr - key);
        s[n][e] = (key <= pr && key >= wl) ? v * kLog2e : -INFINITY;
      }
      mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
      mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
    }
    uint32_t pf[NT][2];
    if (sgm) {
#pragma unroll
      for (int n = 0; n < NT; ++n) {   // a masked score is -inf: exp2(+inf) = inf and the weight is exactly 0
        // the weights are rounded to bf16 for the tensor cores right away: the fast division (2 ulp) is exact enough
        pf[n][0] = pack2(__fdividef(1.f, 1.f + exp2f(-(s[n][0] + sb2))), __fdividef(1.f, 1.f + exp2f(-(s[n][1] + sb2))));
        pf[n][1] = pack2(__fdividef(1.f, 1.f + exp2f(-(s[n][2] + sb2))), __fdividef(1.f, 1.f + exp2f(-(s[n][3] + sb2))));
      }
    } else {
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if (mx0 > mrun[0]) {
      const float c = exp2f(mrun[0] - mx0);   // running maximum -inf: 0, and everything it multiplies is 0
      lrun[0] *= c;
#pragma unroll
      for (int x = 0; x < DT; ++x) { o[x][0] *= c; o[x][1] *= c; }
      mrun[0] = mx0;
    }
    if (mx1 > mrun[1]) {
      const float c = exp2f(mrun[1] - mx1);
      lrun[1] *= c;
#pragma unroll
      for (int x = 0; x < DT; ++x) { o[x][2] *= c; o[x][3] *= c; }
      mrun[1] = mx1;
    }
    const float ms0 = mrun[0] == -INFINITY ? 0.f : mrun[0], ms1 = mrun[1] == -INFINITY ? 0.f : mrun[1];
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const float e0 = exp2f(s[n][0] - ms0), e1 = exp2f(s[n][1] - ms0);
      const float e2 = exp2f(s[n][2] - ms1), e3 = exp2f(s[n][3] - ms1);
      ps0 += e0 + e1; ps1 += e2 + e3;
      pf[n][0] = pack2(e0, e1);
      pf[n][1] = pack2(e2, e3);
    }
    lrun[0] += ps0; lrun[1] += ps1;
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t a0 = pf[2 * kk][0], a1 = pf[2 * kk][1], a2 = pf[2 * kk + 1][0], a3 = pf[2 * kk + 1][1];
#pragma unroll
      for (int dj = 0; dj < DT; dj += 2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(tv + tile_off<VROWB>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dj + (lane >> 4)), b0, b1, b2, b3);
        mma_16816(o[dj], a0, a1, a2, a3, b0, b1);
        mma_16816(o[dj + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();   // the stage is refilled two iterations from now
  }
  float inv[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    float l = lrun[rr];
    l += __shfl_xor_sync(0xffffffffu, l, 1); l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (has_sink) l += exp2f(sk2 - mrun[rr]);   // the sink's logit against the running maximum
    inv[rr] = sgm ? 1.f : 1.f / l;
  }
  const size_t goff = a.g_off + (a.gate_heads ? (size_t)h : (size_t)h * DV);
  const float* g0 = a.g_off >= 0 ? proj + (size_t)(row0 + min(r0, nrows - 1)) * ld + goff : nullptr;
  const float* g1 = a.g_off >= 0 ? proj + (size_t)(row0 + min(r1, nrows - 1)) * ld + goff : nullptr;
  const int gs = a.gate_heads ? 0 : 1;   // one logit per head, or one per output feature
#pragma unroll
  for (int x = 0; x < DT; ++x) {
    const int c = x * 8 + 2 * t4;
    float y0 = o[x][0] * inv[0], y1 = o[x][1] * inv[0], y2 = o[x][2] * inv[1], y3 = o[x][3] * inv[1];
    if (g0) {
      y0 *= 1.f / (1.f + __expf(-g0[gs * c])); y1 *= 1.f / (1.f + __expf(-g0[gs * (c + 1)]));
      y2 *= 1.f / (1.f + __expf(-g1[gs * c])); y3 *= 1.f / (1.f + __expf(-g1[gs * (c + 1)]));
    }
    if (r0 < nrows) *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r0) * a.H + h) * DV + c) = pack2(y0, y1);
    if (r1 < nrows) *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r1) * a.H + h) * DV + c) = pack2(y2, y3);
  }
}

template <int D, int DV>
static cudaError_t launch_tile(__nv_bfloat16* out, const float* q, const float* proj, long long ld, const pieh_bias_attn& a,
                               const pieh_batch& b, cudaStream_t st) {
  constexpr int smem = 2 * (64 * D * 2 + 64 * DV * 2);
  static unsigned long long configured = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(configured >> (dev & 63) & 1)) {
    cudaError_t e = cudaFuncSetAttribute(bias_tile_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured |= 1ull << (dev & 63);
  }
  return launch_k(bias_tile_kernel<D, DV>, dim3(b.n_tiles, a.H), dim3(128), smem, st, out, q, proj, ld, a, b);
}

// the tile kernel serves steps that are mostly prompt portions, over bf16 pages, at the head sizes it is built for
static bool tile_ok(const pieh_bias_attn& a, const pieh_batch& b, int out_dtype) {
  static const bool off = [] { const char* e = getenv("PIE_HYBRID_NO_TILE_ATTN"); return e && e[0] == '1'; }();
  return !off && a.kv_dtype == PIE_DTYPE_BF16 && out_dtype == PIE_DTYPE_BF16 && a.d == a.dv && (a.d == 64 || a.d == 128) &&
         b.n_tiles > 0 && b.tile_seq && b.tile_row && a.H <= 65535 && (long long)b.T >= 16LL * b.n_seq;
}

static bool bias_attn_ok(const pieh_bias_attn* a) {
  return a && a->H > 0 && a->G > 0 && a->H % a->G == 0 && a->d > 0 && a->dv > 0 && a->dv <= 512 && a->d <= 1024 &&
         a->k_pages && a->v_pages && a->temp_every >= 0.0 && a->window >= 0 && a->k_off >= 0 && a->v_off >= 0 &&
         a->rot_dims >= 0 && a->rot_dims <= a->d && (a->rot_dims & 1) == 0 && (a->rot_dims == 0 || a->rot_cs) &&
         (!a->v_mix || a->v_keep) && (a->sigmoid == 0 || a->sigmoid == 1);
}

template <typename KT, typename OT, int NV>
static cudaError_t launch_run_nv(OT* out, const float* q, const float* proj, long long ld, const pieh_bias_attn& a,
                                 const pieh_batch& b, cudaStream_t st) {
  const size_t smem = ((size_t)a.d + (kRunWarps + 1) * (a.dv + 2)) * 4;
  const long long pairs = (long long)b.T * a.H;
  // few (token, head) pairs: clusters of CTAs share a pair's keys until the GPU is covered a few times over
  const long long want = 4LL * num_sms();
  const int cs = pairs * 8 <= want ? 8 : pairs * 4 <= want ? 4 : pairs * 2 <= want ? 2 : 1;
  if (cs == 1) return launch_k(bias_run_kernel<KT, OT, NV, false>, dim3((unsigned)pairs), dim3(kRunWarps * 32), smem, st, out, q, proj, ld, a, b, 1);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(pairs * cs));
  cfg.blockDim = dim3(kRunWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, bias_run_kernel<KT, OT, NV, true>, out, q, proj, ld, a, b, cs);
}

template <typename KT, typename OT>
static cudaError_t launch_run(OT* out, const float* q, const float* proj, long long ld, const pieh_bias_attn& a,
                              const pieh_batch& b, cudaStream_t st) {
  const int nv = (a.dv + 31) / 32;
  if (nv <= 1) return launch_run_nv<KT, OT, 1>(out, q, proj, ld, a, b, st);
  if (nv <= 2) return launch_run_nv<KT, OT, 2>(out, q, proj, ld, a, b, st);
  if (nv <= 4) return launch_run_nv<KT, OT, 4>(out, q, proj, ld, a, b, st);
  if (nv <= 8) return launch_run_nv<KT, OT, 8>(out, q, proj, ld, a, b, st);
  return launch_run_nv<KT, OT, 16>(out, q, proj, ld, a, b, st);
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_bias_attn_prepare(float* q_out, const float* proj, long long ld, const pieh_bias_attn* a,
                                      const pieh_batch* b, void* stream) {
  if (!q_out || !proj || !a || !b) return PIE_ENULL;
  if (!bias_attn_ok(a)) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  count_launch();
  PIEH_DISPATCH_DTYPE(a->kv_dtype, KT, launch_k(bias_prepare_kernel<KT>, dim3(b->T), dim3(256), 0, (cudaStream_t)stream, q_out, proj, ld, *a, *b));
  return status_of(cudaGetLastError());
}

extern "C" int pieh_bias_attn_run(void* out, int out_dtype, const float* q, const float* proj, long long ld,
                                  const pieh_bias_attn* a, const pieh_batch* b, void* stream) {
  if (!out || !q || !a || !b || (a->g_off >= 0 && !proj)) return PIE_ENULL;
  if (!bias_attn_ok(a)) return PIE_EINVAL_SHAPE;
  if (b->T == 0) return PIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  typedef __nv_bfloat16 bf;
  count_launch();
  cudaError_t e;
  if (tile_ok(*a, *b, out_dtype)) {
    e = a->d == 64 ? launch_tile<64, 64>((bf*)out, q, proj, ld, *a, *b, st) : launch_tile<128, 128>((bf*)out, q, proj, ld, *a, *b, st);
    return status_of(e);
  }
  if (a->kv_dtype == PIE_DTYPE_BF16)
    e = out_dtype == PIE_DTYPE_BF16 ? launch_run<bf, bf>((bf*)out, q, proj, ld, *a, *b, st)
                                    : launch_run<bf, float>((float*)out, q, proj, ld, *a, *b, st);
  else
    e = out_dtype == PIE_DTYPE_BF16 ? launch_run<float, bf>((bf*)out, q, proj, ld, *a, *b, st)
                                    : launch_run<float, float>((float*)out, q, proj, ld, *a, *b, st);
  return status_of(e);
}
