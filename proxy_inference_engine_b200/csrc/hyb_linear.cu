// Dense linear layers y = x W^T (+ bias) over unquantized weights, with the epilogues of pie_b200_hybrid.h.
//
// Three kernels behind pieh_linear:
//   * linear_rows_kernel  (M <= 32: decode): a CTA streams 1, 2 or 4 weight rows once with 16-byte loads, its warps cutting K
//     between them, one fp32 accumulator per (activation row, weight row) -- bound by the weight bytes;
//   * linear_umma_kernel  (bf16 x bf16, M > 32, K % 64 == 0: prefill): tcgen05.mma with the fp32 accumulator in
//     tensor memory, both operands brought into 128B-swizzled K-major shared memory by cp.async (hyb_umma.cu);
//   * linear_tile_kernel  (everything else, and every fp32 product): 64 x 64 tiles, fp32 multiply-add on the CUDA cores.
// With bf16 weights the activation is rounded to bf16 first, so the three agree up to the order of the fp32 sums.
#include "hyb_common.cuh"

namespace pieh {


cudaError_t launch_linear_umma(const LinArgs& a, int out_dtype, cudaStream_t st);   // hyb_umma.cu
bool linear_umma_ok(const LinArgs& a, int x_dtype, int w_dtype);
int run_linear(const LinArgs& a, int out_dtype, int x_dtype, int w_dtype, cudaStream_t st);   // picks the kernel

template <typename OT>
__device__ __forceinline__ void lin_store(const LinArgs& a, int m, int n, float y) {
  if (a.bias) y += a.bias[n];
  if (a.epi == PIEH_EPI_RELU2) { y = fmaxf(y, 0.f); y = y * y; }
  else if (a.epi == PIEH_EPI_SOFTCAP) y = a.epi_a * tanhf(y / a.epi_a);
  else if (a.epi == PIEH_EPI_TANH) y = tanhf(y);
  else if (a.epi == PIEH_EPI_XIELU) y = xielu_f(y, a.epi_a, a.epi_b);
  else if (a.epi == PIEH_EPI_SIGMUL) y *= 1.f / (1.f + expf(-a.gate[(size_t)blockIdx.z * a.gate_bs + (size_t)m * a.gate_ld + n]));
  if (a.epi == PIEH_EPI_STREAMS) {
    float* xs = reinterpret_cast<float*>(a.out) + (size_t)m * a.S * a.N + n;
    float old[8];
    for (int s = 0; s < a.S; ++s) old[s] = xs[(size_t)s * a.N];
    for (int u = 0; u < a.S; ++u) {
      float acc = a.outw[u] * y;
      for (int s = 0; s < a.S; ++s) acc = fmaf(a.mix[s * a.S + u], old[s], acc);
      xs[(size_t)u * a.N] = acc;
    }
    return;
  }
  elem<OT>::store(reinterpret_cast<OT*>(a.out) + (size_t)blockIdx.z * a.out_bs + (size_t)m * a.out_ld + n, y);
}

template <typename OT>
__device__ __forceinline__ void lin_store_glu(const LinArgs& a, int m, int n_even, float g, float u) {
  elem<OT>::store(reinterpret_cast<OT*>(a.out) + (size_t)m * a.out_ld + (n_even >> 1), glu_pair(a, g, u));
}

// ------------------------------------------------------------------------------------------------------------------
template <typename XT, typename WT, typename OT>
__global__ void __launch_bounds__(256) linear_tile_kernel(const LinArgs a) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4], Ws[BK][BN + 4];
  pdl_sync();
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  int m0 = blockIdx.y * BM, m_end = a.M;
  const int n0 = blockIdx.x * BN;
  const XT* x = reinterpret_cast<const XT*>(a.x) + (size_t)blockIdx.z * a.x_bs;
  const WT* w = reinterpret_cast<const WT*>(a.w) + (size_t)blockIdx.z * a.w_bs;
  if (a.g_tiles) {   // grouped: this CTA's rows are one expert's run of slots
    if ((int)blockIdx.y >= a.g_tiles[0]) return;
    const int32_t* tl = a.g_tiles + 1 + 3 * blockIdx.y;
    w += (size_t)tl[0] * a.g_wstride;
    m0 = tl[1];
    m_end = tl[1] + tl[2];
  }
  float acc[4][4] = {};
  for (int k0 = 0; k0 < a.K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256, r = e >> 4, c = e & 15;   // r: tile row, c: k within the step
      const int k = k0 + c;
      float xv = 0.f, wv = 0.f;
      if (k < a.K) {
        if (m0 + r < m_end) {
          const int xr = a.g_rows ? a.g_rows[m0 + r] : m0 + r;
          xv = elem<XT>::load(x + (size_t)xr * a.x_ld + k);
          xv = elem<WT>::round(xv);   // bf16 weights: bf16 x bf16 products, exact in fp32
        }
        if (n0 + r < a.N) wv = elem<WT>::load(w + (size_t)(n0 + r) * a.K + k);
      }
      As[c][r] = xv;
      Ws[c][r] = wv;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < BK; ++c) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = As[c][ty * 4 + i]; wv[i] = Ws[c][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
  if (a.epi == PIEH_EPI_GLU) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
        if (m < m_end && n + 1 < a.N) lin_store_glu<OT>(a, m, n, acc[i][j], acc[i][j + 1]);
      }
    return;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < m_end && n < a.N) lin_store<OT>(a, m, n, acc[i][j]);
    }
}

// ------------------------------------------------------------------------------------------------------------------
// M <= 32.  A CTA per R output rows; a lane takes 8 consecutive k per round (16 bytes of bf16, 32 of fp32).
template <typename T> struct vec8;
template <> struct vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
};

template <typename XT, typename WT, typename OT, int MR, int R>
__global__ void __launch_bounds__(256) linear_rows_kernel(const LinArgs a) {
  // one CTA per R consecutive output rows; its 8 warps cut K between them and meet in shared memory
  __shared__ float part[8][MR][R];
  pdl_sync();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * R;
  const XT* x = reinterpret_cast<const XT*>(a.x) + (size_t)blockIdx.z * a.x_bs;
  const WT* w = reinterpret_cast<const WT*>(a.w) + (size_t)blockIdx.z * a.w_bs;
  int mb = 0, M = a.M;   // grouped: one slot per blockIdx.y, with its own expert's matrix
  if (a.g_expert) {
    mb = blockIdx.y;
    M = 1;
    w += (size_t)a.g_expert[mb] * a.g_wstride;
    x += (size_t)(a.g_rows ? a.g_rows[mb] : mb) * a.x_ld;
  }
  float acc[MR][R];
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int r = 0; r < R; ++r) acc[m][r] = 0.f;
#pragma unroll 2
  for (int k = (warp * 32 + lane) * 8; k < a.K; k += 2048) {
    float wv[R][8];
#pragma unroll
    for (int r = 0; r < R; ++r) vec8<WT>::load(w + (size_t)min(n0 + r, a.N - 1) * a.K + k, wv[r]);
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      if (m < M) {
        float xv[8];
        vec8<XT>::load(x + (size_t)m * a.x_ld + k, xv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xr = sizeof(XT) == sizeof(WT) ? xv[i] : elem<WT>::round(xv[i]);   // already in the product type
#pragma unroll
          for (int r = 0; r < R; ++r) acc[m][r] = fmaf(xr, wv[r][i], acc[m][r]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float y = warp_sum(acc[m][r]);
      if (lane == 0) part[warp][m][r] = y;
    }
  __syncthreads();
  if (R % 2 == 0 && a.epi == PIEH_EPI_GLU) {   // the (gate, linear) pairs of this CTA's rows
    constexpr int RP = R > 1 ? R / 2 : 1;
    for (int e = threadIdx.x; e < MR * RP; e += 256) {
      const int m = e / RP, r = 2 * (e - m * RP);
      float g = 0.f, u = 0.f;
#pragma unroll
      for (int wp = 0; wp < 8; ++wp) { g += part[wp][m][r]; u += part[wp][m][r + 1]; }
      if (m < M && n0 + r + 1 < a.N) lin_store_glu<OT>(a, mb + m, n0 + r, g, u);
    }
    return;
  }
  for (int e = threadIdx.x; e < MR * R; e += 256) {
    const int m = e / R, r = e - m * R;
    float y = 0.f;
#pragma unroll
    for (int wp = 0; wp < 8; ++wp) y += part[wp][m][r];
    if (m < M && n0 + r < a.N) lin_store<OT>(a, mb + m, n0 + r, y);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Many rows, few outputs (N <= NMAX <= 32; a router): a warp per activation row, its lanes cutting K in 8-element
// pieces; the whole weight matrix is a few tens of KB and stays in L1 / L2, so the kernel reads x once -- the tensor-core
// tiles would spend a 256-column tile on a handful of columns.
template <typename XT, typename WT, typename OT, int NMAX>
__global__ void __launch_bounds__(256) linear_skinny_kernel(const LinArgs a) {
  pdl_sync();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * 8 + warp;
  if (m >= a.M) return;
  const XT* x = reinterpret_cast<const XT*>(a.x) + (size_t)m * a.x_ld;
  const WT* w = reinterpret_cast<const WT*>(a.w);
  float acc[NMAX];
#pragma unroll
  for (int n = 0; n < NMAX; ++n) acc[n] = 0.f;
  for (int k = lane * 8; k < a.K; k += 256) {
    float xv[8];
    vec8<XT>::load(x + k, xv);
    if (sizeof(XT) != sizeof(WT)) {
#pragma unroll
      for (int i = 0; i < 8; ++i) xv[i] = elem<WT>::round(xv[i]);
    }
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      if (n < a.N) {
        float wv[8];
        vec8<WT>::load(w + (size_t)n * a.K + k, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[n] = fmaf(xv[i], wv[i], acc[n]);
      }
    }
  }
#pragma unroll
  for (int n = 0; n < NMAX; ++n) {
    if (n < a.N) {
      const float y = warp_sum(acc[n]);
      if (lane == 0) lin_store<OT>(a, m, n, y);
    }
  }
}

template <typename XT, typename WT, typename OT>
static cudaError_t launch_typed(const LinArgs& a, cudaStream_t st) {
  const bool vec_ok = a.K % 8 == 0 && a.x_ld % 8 == 0 && (reinterpret_cast<uintptr_t>(a.x) & 31) == 0 &&
                      (reinterpret_cast<uintptr_t>(a.w) & 31) == 0 && a.x_bs % 8 == 0 && a.w_bs % 8 == 0;
  const unsigned nb = (unsigned)a.nb;
  count_launch();
  cudaError_t e = cudaSuccess;
  if (!a.g_tiles && a.nb == 1 && a.M > 32 && a.N <= 32 && vec_ok && a.epi != PIEH_EPI_GLU) {
    const dim3 grid((a.M + 7) / 8);
    if (a.N <= 8) e = launch_k(linear_skinny_kernel<XT, WT, OT, 8>, grid, dim3(256), 0, st, a);
    else if (a.N <= 16) e = launch_k(linear_skinny_kernel<XT, WT, OT, 16>, grid, dim3(256), 0, st, a);
    else e = launch_k(linear_skinny_kernel<XT, WT, OT, 32>, grid, dim3(256), 0, st, a);
  } else if (a.g_tiles) {
    // grouped: few slots -> a CTA per (slot, output rows) streaming that slot's expert; else 64-slot tiles of one expert
    if (a.M <= 32 && vec_ok) {
      const bool wide = (long long)a.N * a.M >= 4 * 4 * num_sms();
      if (wide) e = launch_k(linear_rows_kernel<XT, WT, OT, 1, 4>, dim3((a.N + 3) / 4, a.M), dim3(256), 0, st, a);
      else e = launch_k(linear_rows_kernel<XT, WT, OT, 1, 2>, dim3((a.N + 1) / 2, a.M), dim3(256), 0, st, a);
    } else {
      LinArgs t = a;
      t.g_expert = nullptr;
      const dim3 grid((a.N + 63) / 64, a.M / 64 + (int)a.S);   // S carries the expert count here: the tile list's bound
      e = launch_k(linear_tile_kernel<XT, WT, OT>, grid, dim3(256), 0, st, t);
    }
  } else if (a.M <= 32 && vec_ok) {
    // rows per CTA: enough to amortise the activation loads, few enough that every SM still gets several CTAs
    const bool wide = (long long)a.N * a.nb >= 4 * 4 * num_sms() || a.epi == PIEH_EPI_GLU;   // a gated pair needs an even row count
#define PIEH_ROWS(MR, R) e = launch_k(linear_rows_kernel<XT, WT, OT, MR, R>, dim3((a.N + R - 1) / R, 1, nb), dim3(256), 0, st, a)
    if (a.M <= 1) { if (wide) PIEH_ROWS(1, 2); else PIEH_ROWS(1, 1); }
    else if (a.M <= 4) { if (wide) PIEH_ROWS(4, 4); else PIEH_ROWS(4, 2); }
    else if (a.M <= 8) { if (wide) PIEH_ROWS(8, 4); else PIEH_ROWS(8, 2); }
    else if (a.M <= 16) PIEH_ROWS(16, 2);
    else PIEH_ROWS(32, 2);
#undef PIEH_ROWS
  } else {
    const dim3 grid((a.N + 63) / 64, (a.M + 63) / 64, nb);
    e = launch_k(linear_tile_kernel<XT, WT, OT>, grid, dim3(256), 0, st, a);
  }
  return e;
}

}  // namespace pieh

using namespace pieh;

extern "C" int pieh_linear(void* out, int out_dtype, long long out_ld, const void* x, int x_dtype, long long x_ld,
                           const void* w, int w_dtype, const float* bias, int M, int N, int K, int epilogue, float epi_a,
                           const float* mix, const float* outw, int S, void* stream) {
  if (!out || !x || !w) return PIE_ENULL;
  if (M < 0 || N <= 0 || K <= 0) return PIE_EINVAL_SHAPE;
  if (M == 0) return PIE_OK;
  if (epilogue < 0 || epilogue > PIEH_EPI_STREAMS) return PIE_EUNSUPPORTED;
  if (epilogue == PIEH_EPI_STREAMS && (!mix || !outw || S < 1 || S > 8 || out_dtype != PIE_DTYPE_F32)) return PIE_EINVAL_SHAPE;
  if (epilogue == PIEH_EPI_SOFTCAP && !(epi_a > 0.f)) return PIE_EINVAL_SHAPE;
  LinArgs a{out, out_ld, x, x_ld, w, bias, M, N, K, epilogue, epi_a, mix, outw, S};
  cudaStream_t st = (cudaStream_t)stream;
  return run_linear(a, out_dtype, x_dtype, w_dtype, st);
}

extern "C" int pieh_linear_act(void* out, int out_dtype, long long out_ld, const void* x, int x_dtype, long long x_ld,
                               const void* w, int w_dtype, const float* bias, int M, int N, int K, int act, float act_a,
                               float act_b, void* stream) {
  if (!out || !x || !w) return PIE_ENULL;
  if (M < 0 || N <= 0 || K <= 0) return PIE_EINVAL_SHAPE;
  if (M == 0) return PIE_OK;
  if (act != PIEH_EPI_NONE && act != PIEH_EPI_RELU2 && act != PIEH_EPI_TANH && act != PIEH_EPI_XIELU) return PIE_EUNSUPPORTED;
  LinArgs a{out, out_ld, x, x_ld, w, bias, M, N, K, act, act_a, nullptr, nullptr, 0};
  a.epi_b = act_b;
  return run_linear(a, out_dtype, x_dtype, w_dtype, (cudaStream_t)stream);
}

namespace pieh {
int run_linear(const LinArgs& a, int out_dtype, int x_dtype, int w_dtype, cudaStream_t st) {
  if (w_dtype == PIE_DTYPE_F32 && x_dtype != PIE_DTYPE_F32) return PIE_EINVAL_DTYPE;   // exact mode is fp32 end to end
  // grouped products go to the tensor cores once an expert's run averages a few rows of a 128-slot tile
  if (linear_umma_ok(a, x_dtype, w_dtype) && (!a.g_tiles || a.M >= 8 * a.S)) {
    if (!a.g_tiles) return status_of(launch_linear_umma(a, out_dtype, st));
    LinArgs t = a;          // the tensor-core tiles are 128 slots tall
    t.g_tiles = a.g_tiles128;
    t.g_expert = nullptr;
    return status_of(launch_linear_umma(t, out_dtype, st));
  }
  typedef __nv_bfloat16 bf;
  cudaError_t e;
  if (w_dtype == PIE_DTYPE_F32) {
    e = out_dtype == PIE_DTYPE_F32 ? launch_typed<float, float, float>(a, st) : launch_typed<float, float, bf>(a, st);
  } else if (x_dtype == PIE_DTYPE_F32) {
    e = out_dtype == PIE_DTYPE_F32 ? launch_typed<float, bf, float>(a, st) : launch_typed<float, bf, bf>(a, st);
  } else {
    e = out_dtype == PIE_DTYPE_F32 ? launch_typed<bf, bf, float>(a, st) : launch_typed<bf, bf, bf>(a, st);
  }
  return status_of(e);
}
}  // namespace pieh

extern "C" int pieh_linear_glu(void* out, int out_dtype, long long out_ld, const void* x, int x_dtype, long long x_ld,
                               const void* w, int w_dtype, int M, int N, int K, float alpha, float limit, float up_offset,
                               void* stream) {
  if (!out || !x || !w) return PIE_ENULL;
  if (M < 0 || N <= 0 || K <= 0 || (N & 1) || limit < 0.f) return PIE_EINVAL_SHAPE;
  if (M == 0) return PIE_OK;
  LinArgs a{out, out_ld, x, x_ld, w, nullptr, M, N, K, PIEH_EPI_GLU, limit, nullptr, nullptr, 0};
  a.epi_b = alpha;
  a.epi_c = up_offset;
  return run_linear(a, out_dtype, x_dtype, w_dtype, (cudaStream_t)stream);
}

extern "C" int pieh_moe_linear(void* out, int out_dtype, long long out_ld, const void* x, int x_dtype, long long x_ld,
                               const void* w, int w_dtype, long long w_stride, int P, int N, int K, int gather_rows, int glu,
                               float alpha, float limit, float up_offset, const pieh_moe_plan* p, void* stream) {
  if (!out || !x || !w || !p || !p->tiles64 || !p->tiles128 || !p->slot_row || !p->slot_expert) return PIE_ENULL;
  if (P < 0 || N <= 0 || K <= 0 || glu < 0 || glu > 2 || (glu == 1 && (N & 1)) || p->E < 1 || limit < 0.f) return PIE_EINVAL_SHAPE;
  if (P == 0) return PIE_OK;
  LinArgs a{out, out_ld, x, x_ld, w, nullptr, P, N, K, glu == 1 ? PIEH_EPI_GLU : glu == 2 ? PIEH_EPI_RELU2 : PIEH_EPI_NONE,
            glu == 1 ? limit : 0.f, nullptr, nullptr, p->E};
  a.epi_b = alpha;
  a.epi_c = up_offset;
  a.g_tiles = p->tiles64;
  a.g_tiles128 = p->tiles128;
  a.g_rows = gather_rows ? p->slot_row : nullptr;
  a.g_expert = p->slot_expert;
  a.g_wstride = w_stride;
  return run_linear(a, out_dtype, x_dtype, w_dtype, (cudaStream_t)stream);
}

extern "C" int pieh_linear_batched(void* out, int out_dtype, long long out_ld, long long out_bs, const void* x, int x_dtype,
                                   long long x_ld, long long x_bs, const void* w, int w_dtype, long long w_bs, int nb, int M,
                                   int N, int K, int epilogue, const float* gate, long long gate_ld, long long gate_bs,
                                   void* stream) {
  if (!out || !x || !w) return PIE_ENULL;
  if (M < 0 || N <= 0 || K <= 0 || nb < 1 || nb > 65535) return PIE_EINVAL_SHAPE;
  if (M == 0) return PIE_OK;
  if (epilogue != PIEH_EPI_NONE && epilogue != PIEH_EPI_RELU2 && epilogue != PIEH_EPI_SIGMUL) return PIE_EUNSUPPORTED;
  if (epilogue == PIEH_EPI_SIGMUL && !gate) return PIE_ENULL;
  LinArgs a{out, out_ld, x, x_ld, w, nullptr, M, N, K, epilogue, 0.f, nullptr, nullptr, 0};
  a.x_bs = x_bs; a.w_bs = w_bs; a.out_bs = out_bs;
  a.gate = gate; a.gate_ld = gate_ld; a.gate_bs = gate_bs;
  a.nb = nb;
  return run_linear(a, out_dtype, x_dtype, w_dtype, (cudaStream_t)stream);
}
