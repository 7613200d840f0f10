// Dense bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for prefill-sized steps:
//   y[m, n] = sum_k x[m, k] w[n, k]   (x [M, K] bf16, w [N, K] bf16, fp32 accumulation in tensor memory)
// A CTA owns a BM x 256 tile of y (BM = 256: two 128-row accumulators = all 512 TMEM columns; BM = 128: one).  Per
// 64-element K step and pipeline stage, 256 producer threads bring one 128-byte row piece of x and of w each into the
// 128B-swizzled K-major layout with cp.async (thread t <-> tile row t), make it visible to the async proxy and arrive on
// the stage's mbarrier; one elected lane of a ninth warp issues the tcgen05.mma's (M128 N256 K16) from shared-memory
// descriptors and commits the stage back.  The epilogue reads the accumulators with tcgen05.ld (a warp owns one TMEM
// lane quadrant) and applies pieh_linear's epilogues: bias, relu^2, soft cap, bf16 or fp32 store, or the in-place
// residual-stream update.  Every mbarrier wait is bounded: on expiry the CTA raises an error word the host can read,
// drains its copies, frees its tensor memory and returns.
#include "hyb_common.cuh"
#include "pie_ptx.cuh"
#include "pie_umma.cuh"

namespace pieh {

using pie::smem_u32;


constexpr int kBN = 256, kBK = 64, kProducers = 256, kThreads = kProducers + 32;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr uint32_t IDESC = pie::umma_idesc_bf16_m128(kBN);

__device__ unsigned int g_umma_error = 0;   // 1: a pipeline wait expired

__device__ __forceinline__ bool wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  uint32_t spins = 0;
  while (!pie::mbar_try_wait(bar, parity)) {
    if (++spins > kWaitLimit || *abort_flag) {
      *abort_flag = 1;
      atomicExch(&g_umma_error, 1u);
      return false;
    }
  }
  return true;
}

template <typename OT>
__device__ __forceinline__ void umma_store(const LinArgs& a, int m, int n0, const uint32_t (&v)[32]) {
  if (a.epi == PIEH_EPI_STREAMS) {
    float* xs = reinterpret_cast<float*>(a.out) + (size_t)m * a.S * a.N;
    if (n0 + 32 <= a.N && (a.N & 3) == 0) {   // whole 32-column run, rows 16-byte aligned: four columns at a time
#pragma unroll 2
      for (int q4 = 0; q4 < 8; ++q4) {
        const int n = n0 + 4 * q4;
        float y[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = __uint_as_float(v[4 * q4 + e]) + (a.bias ? a.bias[n + e] : 0.f);
        float4 old[8];
        for (int s = 0; s < a.S; ++s) old[s] = *reinterpret_cast<const float4*>(xs + (size_t)s * a.N + n);
        for (int u = 0; u < a.S; ++u) {
          const float ow = a.outw[u];
          float4 acc = make_float4(ow * y[0], ow * y[1], ow * y[2], ow * y[3]);
          for (int s = 0; s < a.S; ++s) {
            const float mx = a.mix[s * a.S + u];
            acc.x = fmaf(mx, old[s].x, acc.x); acc.y = fmaf(mx, old[s].y, acc.y);
            acc.z = fmaf(mx, old[s].z, acc.z); acc.w = fmaf(mx, old[s].w, acc.w);
          }
          *reinterpret_cast<float4*>(xs + (size_t)u * a.N + n) = acc;
        }
      }
      return;
    }
    for (int q = 0; q < 32; ++q) {
      const int n = n0 + q;
      if (n >= a.N) break;
      float y = __uint_as_float(v[q]);
      if (a.bias) y += a.bias[n];
      float old[8];
      for (int s = 0; s < a.S; ++s) old[s] = xs[(size_t)s * a.N + n];
      for (int u = 0; u < a.S; ++u) {
        float acc = a.outw[u] * y;
        for (int s = 0; s < a.S; ++s) acc = fmaf(a.mix[s * a.S + u], old[s], acc);
        xs[(size_t)u * a.N + n] = acc;
      }
    }
    return;
  }
  if (a.epi == PIEH_EPI_GLU) {   // columns (2 j, 2 j + 1) are a (gate, linear) pair -> output column j
    OT* dst = reinterpret_cast<OT*>(a.out) + (size_t)m * a.out_ld + (n0 >> 1);
    float y[16];
#pragma unroll
    for (int q = 0; q < 16; ++q) y[q] = glu_pair(a, __uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1]));
    if (n0 + 32 <= a.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      if (sizeof(OT) == 4) {
        float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
        for (int q = 0; q < 4; ++q) d4[q] = make_float4(y[4 * q], y[4 * q + 1], y[4 * q + 2], y[4 * q + 3]);
      } else {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int q = 0; q < 2; ++q)
          d4[q] = make_uint4(pie::pack_bf16(y[8 * q], y[8 * q + 1]), pie::pack_bf16(y[8 * q + 2], y[8 * q + 3]),
                             pie::pack_bf16(y[8 * q + 4], y[8 * q + 5]), pie::pack_bf16(y[8 * q + 6], y[8 * q + 7]));
      }
      return;
    }
    for (int q = 0; q < 16; ++q)
      if (n0 + 2 * q + 1 < a.N) elem<OT>::store(dst + q, y[q]);
    return;
  }
  OT* dst = reinterpret_cast<OT*>(a.out) + (size_t)blockIdx.z * a.out_bs + (size_t)m * a.out_ld;
  const float* gate = a.epi == PIEH_EPI_SIGMUL ? a.gate + (size_t)blockIdx.z * a.gate_bs + (size_t)m * a.gate_ld : nullptr;
  float y[32];
  if (gate && n0 + 32 <= a.N && (reinterpret_cast<uintptr_t>(gate + n0) & 15) == 0) {   // the gate logits of a whole run, 16 bytes at a time
#pragma unroll
    for (int q4 = 0; q4 < 8; ++q4) {
      const float4 gq = *reinterpret_cast<const float4*>(gate + n0 + 4 * q4);
      const float gl[4] = {gq.x, gq.y, gq.z, gq.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) y[4 * q4 + e] = __uint_as_float(v[4 * q4 + e]) / (1.f + __expf(-gl[e]));
    }
  } else {
#pragma unroll
    for (int q = 0; q < 32; ++q) {
      const int n = n0 + q;
      float t = __uint_as_float(v[q]);
      if (a.bias && n < a.N) t += a.bias[n];
      if (a.epi == PIEH_EPI_RELU2) { t = fmaxf(t, 0.f); t = t * t; }
      else if (a.epi == PIEH_EPI_SOFTCAP) t = a.epi_a * tanhf(t / a.epi_a);
      else if (a.epi == PIEH_EPI_TANH) t = tanhf(t);
      else if (a.epi == PIEH_EPI_XIELU) t = xielu_f(t, a.epi_a, a.epi_b);
      else if (a.epi == PIEH_EPI_SIGMUL && n < a.N) t *= 1.f / (1.f + __expf(-gate[n]));
      y[q] = t;
    }
  }
  if (n0 + 32 <= a.N && (reinterpret_cast<uintptr_t>(dst + n0) & 15) == 0) {
    if (sizeof(OT) == 4) {
      float4* d4 = reinterpret_cast<float4*>(dst + n0);
#pragma unroll
      for (int q = 0; q < 8; ++q) d4[q] = make_float4(y[4 * q], y[4 * q + 1], y[4 * q + 2], y[4 * q + 3]);
    } else {
      uint4* d4 = reinterpret_cast<uint4*>(dst + n0);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        d4[q] = make_uint4(pie::pack_bf16(y[8 * q], y[8 * q + 1]), pie::pack_bf16(y[8 * q + 2], y[8 * q + 3]),
                           pie::pack_bf16(y[8 * q + 4], y[8 * q + 5]), pie::pack_bf16(y[8 * q + 6], y[8 * q + 7]));
    }
    return;
  }
  for (int q = 0; q < 32; ++q)
    if (n0 + q < a.N) elem<OT>::store(dst + n0 + q, y[q]);
}

// S stages: <256, 3> and <128, 4>, one CTA per SM.  (Two 128-row CTAs per SM with 2 stages each, so that one's epilogue
// runs under the other's main loop, measured 20-30 % slower than either.)
template <int BM, int S, typename OT>
__global__ void __launch_bounds__(kThreads, 1) linear_umma_kernel(const __grid_constant__ LinArgs a) {
  constexpr int NACC = BM / 128;
  constexpr int LAG = S == 4 ? 2 : 1;   // k-steps of loads in flight behind the one the tensor core reads
  constexpr int A_STAGE = BM * kBK * 2, B_STAGE = kBN * kBK * 2;
  constexpr int TMEM_COLS = NACC * kBN;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[S], empty_bar[S], accum_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  pdl_sync();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smA = base, smB = base + S * A_STAGE;
  const int n0 = blockIdx.x * kBN;
  int m0 = blockIdx.y * BM, m_end = a.M;
  const __nv_bfloat16* wmat = reinterpret_cast<const __nv_bfloat16*>(a.w) + (size_t)blockIdx.z * a.w_bs;
  if (a.g_tiles) {   // grouped: this CTA's rows are one expert's run of slots (the whole CTA leaves before anything is set up)
    if ((int)blockIdx.y >= a.g_tiles[0]) return;
    const int32_t* tl = a.g_tiles + 1 + 3 * blockIdx.y;
    wmat += (size_t)tl[0] * a.g_wstride;
    m0 = tl[1];
    m_end = tl[1] + tl[2];
  }
  const int nk = a.K / kBK;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) { pie::mbar_init(&full_bar[s], kProducers); pie::mbar_init(&empty_bar[s], 1); }
    pie::mbar_init(&accum_bar, 1);
    abort_flag = 0;
    pie::fence_mbar_init();
  }
  if (warp == kProducers / 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "n"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_slot;

  if (warp < kProducers / 32) {
    const int t = tid;
    const uint32_t swz = (uint32_t)(t & 7);
    const __nv_bfloat16* wsrc = wmat + (size_t)min(n0 + t, a.N - 1) * a.K;
    const int xslot = min(m0 + min(t, BM - 1), m_end - 1);
    const __nv_bfloat16* xsrc = reinterpret_cast<const __nv_bfloat16*>(a.x) + (size_t)blockIdx.z * a.x_bs +
                                (size_t)(a.g_rows ? a.g_rows[xslot] : xslot) * a.x_ld;
    bool alive = true;
    for (int kb = 0; kb < nk + LAG && alive; ++kb) {
      if (kb < nk) {
        const int s = kb % S, it = kb / S;
        if (it > 0) alive = wait_bounded(&empty_bar[s], (uint32_t)(it - 1) & 1, &abort_flag);
        if (alive) {
          if (t < BM) {
            const uint32_t dA = smA + s * A_STAGE + t * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) pie::cp_async16(dA + ((c ^ swz) << 4), xsrc + kb * kBK + c * 8);
          }
          const uint32_t dB = smB + s * B_STAGE + t * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) pie::cp_async16(dB + ((c ^ swz) << 4), wsrc + kb * kBK + c * 8);
        }
      }
      pie::cp_async_commit();
      if (kb >= LAG && alive) {
        pie::cp_async_wait<LAG>();
        pie::fence_proxy_async();
        pie::mbar_arrive(&full_bar[(kb - LAG) % S]);
      }
    }
    pie::cp_async_wait<0>();
    // ---- epilogue: this warp's TMEM lane quadrant
    if (alive) alive = wait_bounded(&accum_bar, 0, &abort_flag);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (alive) {
      const int quad = warp & 3;
      const int h = NACC == 2 ? (warp >> 2) : 0;
      const int c_lo = NACC == 2 ? 0 : (warp >> 2) * (kBN / 64), c_hi = NACC == 2 ? kBN / 32 : c_lo + kBN / 64;
      const int row = m0 + h * 128 + quad * 32 + lane;
#pragma unroll 1
      for (int c = c_lo; c < c_hi; ++c) {
        uint32_t v[32];
        pie::tmem_ld32(tmem + (uint32_t)(h * kBN + c * 32) + ((uint32_t)(quad * 32) << 16), v);
        if (row < m_end && n0 + c * 32 < a.N) umma_store<OT>(a, row, n0 + c * 32, v);
      }
    }
  } else {
    bool alive = true;
    for (int kb = 0; kb < nk && alive; ++kb) {
      const int s = kb % S;
      alive = wait_bounded(&full_bar[s], (uint32_t)(kb / S) & 1, &abort_flag);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0 && alive) {
        const uint64_t db0 = pie::umma_desc_sw128(smB + s * B_STAGE);
#pragma unroll
        for (int h = 0; h < NACC; ++h) {
          const uint64_t da0 = pie::umma_desc_sw128(smA + s * A_STAGE + h * 128 * 128);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4)
            pie::umma_bf16(tmem + h * kBN, da0 + 2 * k4, db0 + 2 * k4, IDESC, (kb > 0 || k4 > 0) ? 1u : 0u);
        }
        pie::umma_commit(&empty_bar[s]);
        if (kb == nk - 1) pie::umma_commit(&accum_bar);
      }
      __syncwarp();
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kProducers / 32)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(TMEM_COLS) : "memory");
}

bool linear_umma_ok(const LinArgs& a, int x_dtype, int w_dtype) {
  static const bool off = [] { const char* e = getenv("PIE_HYBRID_NO_UMMA"); return e && e[0] == '1'; }();
  if (off) return false;
  if (!a.g_tiles && a.N <= 32 && a.K % 8 == 0 && (reinterpret_cast<uintptr_t>(a.w) & 31) == 0 &&
      (reinterpret_cast<uintptr_t>(a.x) & 31) == 0 && a.epi != PIEH_EPI_GLU)
    return false;   // a handful of output columns: linear_skinny_kernel reads x once instead of filling 256-column tiles
  if (a.x_bs % 8 || a.w_bs % 8) return false;   // every product's operands start on a 16-byte boundary
  return x_dtype == PIE_DTYPE_BF16 && w_dtype == PIE_DTYPE_BF16 && a.M > 32 && a.K % kBK == 0 && a.x_ld % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.w) & 15) == 0;
}

template <int BM, int S, typename OT>
static cudaError_t launch_bm(const LinArgs& a, cudaStream_t st) {
  constexpr size_t smem = (size_t)S * (BM * kBK * 2 + kBN * kBK * 2) + 1024;
  static unsigned long long configured = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(configured >> (dev & 63) & 1)) {
    cudaError_t e = cudaFuncSetAttribute(linear_umma_kernel<BM, S, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured |= 1ull << (dev & 63);
  }
  // grouped: blockIdx.y walks the list of <= 128-slot tiles, whose length is only known on the device (S = experts)
  const dim3 grid((a.N + kBN - 1) / kBN, a.g_tiles ? a.M / 128 + a.S : (a.M + BM - 1) / BM, a.nb);
  count_launch();
  linear_umma_kernel<BM, S, OT><<<grid, kThreads, smem, st>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_linear_umma(const LinArgs& a, int out_dtype, cudaStream_t st) {
  // 256-row tiles halve the weight traffic per flop and measured faster down to half a wave of tiles (M 2048 x N 4096:
  // 390 against 262 TFLOP/s); below that the 128-row tiles spread the work over more SMs
  const long long tiles256 = (long long)((a.N + kBN - 1) / kBN) * ((a.M + 255) / 256) * a.nb;
  static const int force = [] { const char* e = getenv("PIE_HYBRID_UMMA_TILE"); return e ? atoi(e) : 0; }();   // tuning
  int variant = a.M > 128 && 2 * tiles256 >= num_sms() ? 256 : 128;
  if (force == 128 || force == 256) variant = force;
  if (a.g_tiles) variant = 128;
#define PIEH_UMMA(OT) (variant == 256 ? launch_bm<256, 3, OT>(a, st) : launch_bm<128, 4, OT>(a, st))
  if (out_dtype == PIE_DTYPE_BF16) return PIEH_UMMA(__nv_bfloat16);
  return PIEH_UMMA(float);
#undef PIEH_UMMA
}

}  // namespace pieh

extern "C" unsigned int pieh_pipeline_error(void) {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, pieh::g_umma_error, sizeof(v));
  return v;
}
