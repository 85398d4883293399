// Causal flash attention forward on tcgen05 / TMEM for sm_100a: packed variable-length
// documents, MHA and GQA, head_dim 128, bf16 in/out, fp32 softmax.
//
// One CTA per (128-query tile, query head); 192 threads:
//   warp 0     TMA: Q tile once, then K and V tiles (128 keys) through 2-stage rings
//   warp 1     one thread issues S = Q·Kᵀ (128x128x128) into one of two TMEM S buffers and
//              O += P·V (P from shared memory, V read in place as an MN-major operand)
//   warps 2-5  softmax: thread r owns query row r (its TMEM lane), so row max / row sum need
//              no shuffles; exp2 with the scale folded in; P is written as bf16 into swizzled
//              shared memory; the O accumulator in TMEM is rescaled only when a row maximum grew
//              by more than 2^8 (stale-max trick: the final 1/l normalisation makes it exact).
// S(j+1) is issued before softmax(j) finishes, so tensor-core work overlaps the exponentials.
// Documents: row_start[t] is the first token of the document that token t belongs to; key j is
// visible to query i iff row_start[i] <= j <= i, so tiles may straddle document boundaries.
//
// Replaces flash_attn_varlen_{qkv,kv}packed_func of the reference
// (llm/models/mg_models/llama/transformer.py:65-143).
#include "common.cuh"
#include "sm100.cuh"

namespace ell {
using namespace sm100;

constexpr int kFaThreads = 192;
constexpr int kFaM = 128, kFaN = 128, kFaD = 128;
constexpr int kFaTileBytes = 128 * 128 * 2;  // 32 KiB: Q, K, V and P tiles are all 128x128 bf16
constexpr int kFaSmemBytes = 6 * kFaTileBytes + 1024 + 256;
constexpr float kFaRescaleThreshold = 8.0f;   // log2 units

struct FaShared {
  uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], p_full, pv_done;
  uint32_t tmem_base;
  int abort_flag;
  int sm_abort;
};

enum FaErr { kFaErrProducer = 11, kFaErrMma = 12, kFaErrSoftmax = 13 };

__global__ void __launch_bounds__(kFaThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ out,
                 float* __restrict__ lse, const int* __restrict__ row_start, int T, int Hq, int Hk,
                 float scale_log2, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kFaTileBytes;          // 2 stages
  uint8_t* sV = smem + 3 * kFaTileBytes;      // 2 stages
  uint8_t* sP = smem + 5 * kFaTileBytes;
  FaShared* sh = reinterpret_cast<FaShared*>(smem + 6 * kFaTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qtiles = (T + kFaM - 1) / kFaM;
  const int qt = n_qtiles - 1 - blockIdx.x;   // heaviest (latest) tiles first
  const int h = blockIdx.y;
  const int kvh = h / (Hq / Hk);
  const int q0 = qt * kFaM;
  const int q_last = min(q0 + kFaM, T) - 1;
  const int kv_lo = row_start[q0];
  const int kv_hi = q_last + 1;
  const int n_kv = (kv_hi - kv_lo + kFaN - 1) / kFaN;
  const int max_row_start = row_start[q_last];

  if (threadIdx.x == 0) {
    mbar_init(&sh->q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->k_full[s], 1);
      mbar_init(&sh->v_full[s], 1);
      mbar_init(&sh->k_empty[s], 1);
      mbar_init(&sh->v_empty[s], 1);
      mbar_init(&sh->s_full[s], 1);
    }
    mbar_init(&sh->p_full, 128);
    mbar_init(&sh->pv_done, 1);
    sh->abort_flag = 0;
    sh->sm_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) tmem_alloc<512>(&sh->tmem_base);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const uint32_t tmem_o = tmem_base + 256;
  volatile int* abort_flag = &sh->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(&sh->q_full, kFaTileBytes);
      tma_load_2d(sQ, &tmQ, &sh->q_full, h * kFaD, q0);
      tma_load_2d(sQ + kFaTileBytes / 2, &tmQ, &sh->q_full, h * kFaD + 64, q0);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int k0 = kv_lo + j * kFaN;
        if (!mbar_wait(&sh->k_empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(&sh->k_full[s], kFaTileBytes);
        tma_load_2d(sK + s * kFaTileBytes, &tmK, &sh->k_full[s], kvh * kFaD, k0);
        tma_load_2d(sK + s * kFaTileBytes + kFaTileBytes / 2, &tmK, &sh->k_full[s], kvh * kFaD + 64, k0);
        if (!mbar_wait(&sh->v_empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(&sh->v_full[s], kFaTileBytes);
        tma_load_2d(sV + s * kFaTileBytes, &tmV, &sh->v_full[s], kvh * kFaD, k0);
        tma_load_2d(sV + s * kFaTileBytes + kFaTileBytes / 2, &tmV, &sh->v_full[s], kvh * kFaD + 64, k0);
      }
      if (!ok) {
        sh->abort_flag = 1;
        atomicCAS(err, 0, kFaErrProducer);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);
      bool ok = mbar_wait(&sh->q_full, 0, abort_flag);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&sh->k_full[s], (j >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * kFaTileBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * (kFaTileBytes / 2) + (k & 3) * 32;
          umma_bf16(tmem_base + s * 128, make_smem_desc(q_addr + off, 16, 1024), make_smem_desc(k_addr + off, 16, 1024),
                    idesc_s, k != 0);
        }
        umma_commit(&sh->s_full[s]);
        umma_commit(&sh->k_empty[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          if (!issue_s(j + 1)) { ok = false; break; }
        }
        const int s = j & 1;
        if (!mbar_wait(&sh->p_full, j & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&sh->v_full[s], (j >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * kFaTileBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t a_off = (k >> 2) * (kFaTileBytes / 2) + (k & 3) * 32;
          umma_bf16(tmem_o, make_smem_desc(p_addr + a_off, 16, 1024),
                    make_smem_desc(v_addr + k * 2048, kFaTileBytes / 2, 1024), idesc_o, (j | k) != 0);
        }
        umma_commit(&sh->pv_done);
        umma_commit(&sh->v_empty[s]);
      }
      if (!ok) {
        sh->abort_flag = 1;
        atomicCAS(err, 0, kFaErrMma);
      }
    }
  } else {
    // ---------------- softmax / correction / epilogue: thread <-> query row ----------------
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int row = q0 + r;
    const bool row_valid = row < T;
    const int my_start = row_valid ? row_start[row] : 0x7fffffff;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    float m_used = -1e30f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int sb = j & 1;
      if (!mbar_wait(&sh->s_full[sb], (j >> 1) & 1, abort_flag)) sh->sm_abort = 1;
      named_bar_sync(1, 128);
      if (*(volatile int*)&sh->sm_abort) { ok = false; break; }
      tc_fence_after();
      const int k0 = kv_lo + j * kFaN;
      const bool need_mask = (k0 + kFaN - 1 > q0) || (k0 < max_row_start);
      const uint32_t t_s = tmem_base + lane_off + sb * 128;
      // pass 1: row maximum (log2 domain)
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_s + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float t = __uint_as_float(v[i]) * scale_log2;
          if (need_mask) {
            const int kidx = k0 + c * 32 + i;
            if (kidx > row || kidx < my_start) t = -INFINITY;
          }
          mx = fmaxf(mx, t);
        }
      }
      const float m_new = fmaxf(m_used, mx);
      const bool grow = (m_new - m_used) > kFaRescaleThreshold;
      const bool any_grow = __any_sync(0xffffffffu, grow);
      // P(j) overwrites the tile PV(j-1) reads, and a rescale touches O: wait for PV(j-1)
      if (j > 0) {
        if (!mbar_wait(&sh->pv_done, (j - 1) & 1, abort_flag)) sh->sm_abort = 1;
      }
      if (any_grow) {
        const float alpha = grow ? exp2f(m_used - m_new) : 1.f;
        if (grow) {
          m_used = m_new;
          l *= alpha;
        }
        if (j > 0) {
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_o + lane_off + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(tmem_o + lane_off + c * 32, v);
          }
          tmem_st_wait();
        }
      }
      // pass 2: P = exp2(t - m_used) -> bf16 -> swizzled smem; row sum
      float psum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_s + c * 32, v);
        tmem_ld_wait();
        uint8_t* atom = sP + (c >> 1) * (kFaTileBytes / 2) + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float p[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float t = __uint_as_float(v[g * 8 + i]) * scale_log2;
            if (need_mask) {
              const int kidx = k0 + c * 32 + g * 8 + i;
              if (kidx > row || kidx < my_start) t = -INFINITY;
            }
            p[i] = exp2f(t - m_used);
            psum += p[i];
          }
          bf16x8 pk = pack8(p);
          const int chunk = (c & 1) * 4 + g;
          *reinterpret_cast<bf16x8*>(atom + ((chunk ^ (r & 7)) << 4)) = pk;
        }
      }
      l += psum;
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&sh->p_full);
    }
    // ---------------- epilogue: O / l -> bf16 -> global; LSE ----------------
    if (ok) {
      if (!mbar_wait(&sh->pv_done, (n_kv - 1) & 1, abort_flag)) sh->sm_abort = 1;
    }
    named_bar_sync(1, 128);
    if (!*(volatile int*)&sh->sm_abort) {
      tc_fence_after();
      const float inv_l = row_valid ? 1.f / l : 0.f;
      __nv_bfloat16* orow = out + ((size_t)row * Hq + h) * kFaD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_o + lane_off + c * 32, v);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[g * 8 + i]) * inv_l;
            *reinterpret_cast<bf16x8*>(orow + c * 32 + g * 8) = pack8(f);
          }
        }
      }
      if (row_valid) lse[(size_t)h * T + row] = m_used * 0.6931471805599453f + logf(l);
    } else if (threadIdx.x == 64) {
      sh->abort_flag = 1;
      atomicCAS(err, 0, kFaErrSoftmax);
    }
  }

  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<512>(tmem_base);
  }
}

int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                      uint32_t box_inner, uint32_t box_outer);

}  // namespace ell

using namespace ell;

// q [T, Hq, 128] / k, v [T, Hk, 128] bf16 with row strides (in elements) q_stride / kv_stride (views
// into the packed QKV GEMM output are fine); out [T, Hq, 128] contiguous; lse [Hq, T] fp32;
// row_start [T] int32 (document start of every token).  Causal.
ELL_API int ell_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* row_start,
                               int T, int Hq, int Hk, int q_stride, int kv_stride, float scale, int* err,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (Hq % Hk) return -2;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_bf16_2d(&tq, q, (uint64_t)Hq * kFaD, (uint64_t)T, (uint64_t)q_stride * 2, 64, 128);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tk, k, (uint64_t)Hk * kFaD, (uint64_t)T, (uint64_t)kv_stride * 2, 64, 128);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tv, v, (uint64_t)Hk * kFaD, (uint64_t)T, (uint64_t)kv_stride * 2, 64, 128);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFaSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((T + kFaM - 1) / kFaM, Hq);
  flash_fwd_kernel<<<grid, kFaThreads, kFaSmemBytes, stream>>>(tq, tk, tv, (__nv_bfloat16*)out, lse, row_start, T, Hq,
                                                               Hk, scale * 1.4426950408889634f, err);
  return launch_status();
}
