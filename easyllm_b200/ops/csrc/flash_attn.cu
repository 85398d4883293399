// Causal flash attention forward on tcgen05 / TMEM for sm_100a: packed variable-length
// documents, MHA and GQA, head_dim 128, bf16 in/out, fp32 softmax.
//
// One CTA per (pair of adjacent 128-query tiles, query head); 320 threads:
//   warp 0     TMA: both Q tiles once, then K tiles (128 keys) through a 2-stage ring and V tiles one at a time
//   warp 1     one thread issues, for every key tile j, S_t = Q_t·K_jᵀ (128x128x128) for both query tiles and
//              O_t += P_t·V_j (P from shared memory, V read in place as an MN-major operand).
//              TMEM columns: S_0 0-127, S_1 128-255, O_0 256-383, O_1 384-511.
//   warps 2-5 / 6-9   one softmax group per query tile: thread r owns query row r (its TMEM lane), so row
//              max / row sum need no shuffles.  The whole S row is pulled into registers at once (the S columns
//              are handed back to the tensor core immediately, so S_t(j+1) overlaps the exponentials of step j),
//              exp2 with the scale folded into one FMA, P written as bf16 into swizzled shared memory; the O
//              accumulator is rescaled only when a row maximum grew by more than 2^8 (stale-max trick: the final
//              1/l normalisation makes it exact).
// Two groups per SM keep two warps on every scheduler, so one group's TMEM-load and MUFU latencies hide behind
// the other's arithmetic, and each K/V tile fetched serves 256 queries.
// Documents: row_start[t] is the first token of the document that token t belongs to; key j is
// visible to query i iff row_start[i] <= j <= i, so tiles may straddle document boundaries.
// ALiBi: with per-head slopes the score of (query i, key j) gets the bias slope_h * (j - i) before the softmax
// (llm/models/hf_models/baichuan2/model_13b/modeling_baichuan.py:63-73 builds the same bias as a mask tensor).
//
// Replaces flash_attn_varlen_{qkv,kv}packed_func of the reference
// (llm/models/mg_models/llama/transformer.py:65-143).
#include "common.cuh"
#include "sm100.cuh"

namespace ell {
using namespace sm100;

constexpr int kFaThreads = 320;
constexpr int kFaM = 128, kFaN = 128, kFaD = 128;
constexpr int kFaTileBytes = 128 * 128 * 2;  // 32 KiB: Q, K, V and P tiles are all 128x128 bf16
constexpr int kFaSmemBytes = 7 * kFaTileBytes + 1024 + 512;   // Q x2, K x2, V, P x2
constexpr float kFaRescaleThreshold = 8.0f;   // log2 units

struct FaShared {
  uint64_t q_full, k_full[2], k_empty[2], v_full, v_empty, s_full[2], s_free[2], p_full[2], pv_done[2];
  uint32_t tmem_base;
  int abort_flag;
};

enum FaErr { kFaErrProducer = 11, kFaErrMma = 12, kFaErrSoftmax = 13 };

// Optional timeline of the first CTA (clock64 stamps per role, step and stage), compiled in with -DELL_FA_TRACE.
#ifdef ELL_FA_TRACE
__device__ long long* g_fa_trace = nullptr;   // [3 roles][64 steps][8 stages]
#define FA_TRACE(role, it, slot)                                                             \
  do {                                                                                       \
    if (blockIdx.x == 0 && blockIdx.y == 0 && g_fa_trace && (it) < 64)                       \
      g_fa_trace[(((role) * 64 + (it)) << 3) + (slot)] = clock64();                          \
  } while (0)
#else
#define FA_TRACE(role, it, slot)
#endif

// registers are granted per 4 warps: 10 warps count as 12, which caps a thread at 168 registers
// Tile plan of the forward kernel, __host__ __device__ so that ell_flash_fwd_plan can run the same arithmetic on the
// host for a CPU test.  A query tile starting at row `first` walks key tiles of kFaN keys from kv_lo (the document
// start of the first row of the CTA's tile pair) up to the tile's last row.
__host__ __device__ __forceinline__ int fa_num_kv_tiles(int first, int T, int kv_lo) {
  const int last = (first + kFaM < T ? first + kFaM : T) - 1;
  return first < T ? (last + 1 - kv_lo + kFaN - 1) / kFaN : 0;
}

// A key tile starting at k0 needs no per-element mask when every key in it precedes (or is) the tile's first query
// row and no row of the query tile starts its document after k0.
__host__ __device__ __forceinline__ bool fa_tile_needs_mask(int k0, int tile_first, int max_row_start) {
  return (k0 + kFaN - 1 > tile_first) || (k0 < max_row_start);
}

__global__ void __launch_bounds__(kFaThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ out,
                 float* __restrict__ lse, const int* __restrict__ row_start, int T, int Hq, int Hk,
                 float scale_log2, const float* __restrict__ alibi_slopes, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                          // 2 query tiles
  uint8_t* sK = smem + 2 * kFaTileBytes;       // 2 stages
  uint8_t* sV = smem + 4 * kFaTileBytes;       // 1 stage
  uint8_t* sP = smem + 5 * kFaTileBytes;       // 2 query tiles
  FaShared* sh = reinterpret_cast<FaShared*>(smem + 7 * kFaTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_pairs = (T + 2 * kFaM - 1) / (2 * kFaM);
  const int pair = n_pairs - 1 - blockIdx.x;   // heaviest (latest) pairs first
  const int h = blockIdx.y;
  const int kvh = h / (Hq / Hk);
  const int q0 = pair * 2 * kFaM;              // first query row of tile 0; tile 1 starts at q0 + 128
  const int kv_lo = row_start[q0];
  // key tiles each query tile walks: tile t covers keys kv_lo .. last row of the tile
  int n_kv[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) n_kv[t] = fa_num_kv_tiles(q0 + t * kFaM, T, kv_lo);
  const int n_kv_max = max(n_kv[0], n_kv[1]);

  if (threadIdx.x == 0) {
    mbar_init(&sh->q_full, 1);
    mbar_init(&sh->v_full, 1);
    mbar_init(&sh->v_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->k_full[s], 1);
      mbar_init(&sh->k_empty[s], 1);
      mbar_init(&sh->s_full[s], 1);
      mbar_init(&sh->s_free[s], 128);
      mbar_init(&sh->p_full[s], 128);
      mbar_init(&sh->pv_done[s], 1);
    }
    sh->abort_flag = *(volatile int*)err;      // an earlier CTA already failed: do not wait on anything
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
  const bool dead_on_arrival = sh->abort_flag != 0;
  volatile int* abort_flag = &sh->abort_flag;

  if (dead_on_arrival) {
    // fall through to the common exit: nothing was issued
  } else if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(&sh->q_full, 2 * kFaTileBytes);
#pragma unroll
      for (int t = 0; t < 2; ++t) {            // rows past T are zero-filled by the TMA unit
        tma_load_2d(sQ + t * kFaTileBytes, &tmQ, &sh->q_full, h * kFaD, q0 + t * kFaM);
        tma_load_2d(sQ + t * kFaTileBytes + kFaTileBytes / 2, &tmQ, &sh->q_full, h * kFaD + 64, q0 + t * kFaM);
      }
      // K runs one tile ahead of V: K(j+1) is requested as soon as S(j-1) released its stage, before the
      // loader blocks on the single V stage (free only once PV(j-1) is done)
      auto load_k = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&sh->k_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) return false;
        mbar_expect_tx(&sh->k_full[s], kFaTileBytes);
        tma_load_2d(sK + s * kFaTileBytes, &tmK, &sh->k_full[s], kvh * kFaD, kv_lo + j * kFaN);
        tma_load_2d(sK + s * kFaTileBytes + kFaTileBytes / 2, &tmK, &sh->k_full[s], kvh * kFaD + 64, kv_lo + j * kFaN);
        return true;
      };
      if (n_kv_max > 0) ok = load_k(0);
      for (int j = 0; j < n_kv_max && ok; ++j) {
        const int k0 = kv_lo + j * kFaN;
        if (j + 1 < n_kv_max && !load_k(j + 1)) { ok = false; break; }
        if (!mbar_wait(&sh->v_empty, (j & 1) ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(&sh->v_full, kFaTileBytes);
        tma_load_2d(sV, &tmV, &sh->v_full, kvh * kFaD, k0);
        tma_load_2d(sV + kFaTileBytes / 2, &tmV, &sh->v_full, kvh * kFaD + 64, k0);
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
      const uint32_t v_addr = smem_u32(sV);
      // S_t(j) = Q_t K_j^T for both query tiles that still walk key tile j
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&sh->k_full[s], (j >> 1) & 1, abort_flag)) return false;
        const uint32_t k_addr = smem_u32(sK + s * kFaTileBytes);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= n_kv[t]) continue;
          // the softmax group has pulled S_t(j-1) into registers
          if (j > 0 && !mbar_wait(&sh->s_free[t], (j - 1) & 1, abort_flag)) return false;
          tc_fence_after();
          const uint32_t q_addr = smem_u32(sQ + t * kFaTileBytes);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = (k >> 2) * (kFaTileBytes / 2) + (k & 3) * 32;
            umma_bf16(tmem_base + t * 128, make_smem_desc(q_addr + off, 16, 1024),
                      make_smem_desc(k_addr + off, 16, 1024), idesc_s, k != 0);
          }
          umma_commit(&sh->s_full[t]);
        }
        umma_commit(&sh->k_empty[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv_max && ok; ++j) {
        FA_TRACE(0, j, 0);
        if (j + 1 < n_kv_max && !issue_s(j + 1)) { ok = false; break; }
        FA_TRACE(0, j, 1);
        if (!mbar_wait(&sh->v_full, j & 1, abort_flag)) { ok = false; break; }
        FA_TRACE(0, j, 2);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= n_kv[t] || !ok) continue;
          if (!mbar_wait(&sh->p_full[t], j & 1, abort_flag)) { ok = false; continue; }
          FA_TRACE(0, j, 3 + t);
          tc_fence_after();
          const uint32_t p_addr = smem_u32(sP + t * kFaTileBytes);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t a_off = (k >> 2) * (kFaTileBytes / 2) + (k & 3) * 32;
            umma_bf16(tmem_base + 256 + t * 128, make_smem_desc(p_addr + a_off, 16, 1024),
                      make_smem_desc(v_addr + k * 2048, kFaTileBytes / 2, 1024), idesc_o, (j | k) != 0);
          }
          umma_commit(&sh->pv_done[t]);
        }
        umma_commit(&sh->v_empty);
        FA_TRACE(0, j, 5);
      }
      if (!ok) {
        sh->abort_flag = 1;
        atomicCAS(err, 0, kFaErrMma);
      }
    }
  } else {
    // ---------------- softmax / correction / epilogue: one group per query tile ----------------
    const int t = (warp - 2) >> 2;               // query tile of this group
    const int quad = warp & 3;                   // TMEM lane quadrant this warp may access
    const int r = quad * 32 + lane;
    const int row = q0 + t * kFaM + r;
    const bool row_valid = row < T;
    const int my_start = row_valid ? row_start[row] : 0x7fffffff;
    const int tile_first = q0 + t * kFaM;
    const int max_row_start = n_kv[t] > 0 ? row_start[min(tile_first + kFaM, T) - 1] : 0;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const uint32_t t_s = tmem_base + lane_off + t * 128;
    const uint32_t t_o = tmem_base + lane_off + 256 + t * 128;
    uint8_t* p_row = sP + t * kFaTileBytes + r * 128;
    const int sw = r & 7;
    float m_used = -1e30f, l = 0.f;
    // ALiBi bias in units of the raw score: (slope / scale) * (key - query), so that score * scale_log2 carries it
    const float alibi_s = alibi_slopes != nullptr ? alibi_slopes[h] * 1.4426950408889634f / scale_log2 : 0.f;
    bool ok = true;
    auto fail = [&]() {
      ok = false;
      sh->abort_flag = 1;
      atomicCAS(err, 0, kFaErrSoftmax);
    };
    const int my_n = n_kv[t];
    for (int j = 0; j < my_n; ++j) {
      if (threadIdx.x == 64) FA_TRACE(1, j, 0);
      if (!mbar_wait(&sh->s_full[t], j & 1, abort_flag)) fail();
      if (threadIdx.x == 64) FA_TRACE(1, j, 1);
      tc_fence_after();
      uint32_t s[128];
      tmem_ld_32x32(t_s, s);
      tmem_ld_32x32(t_s + 32, s + 32);
      tmem_ld_32x32(t_s + 64, s + 64);
      tmem_ld_32x32(t_s + 96, s + 96);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&sh->s_free[t]);               // S_t(j+1) may overwrite the columns now
      if (threadIdx.x == 64) FA_TRACE(1, j, 2);
      const int k0 = kv_lo + j * kFaN;
      const bool need_mask = fa_tile_needs_mask(k0, tile_first, max_row_start);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const int kidx = k0 + i;
          if (kidx > row || kidx < my_start) s[i] = 0xff800000u;   // -inf
        }
      }
      if (alibi_slopes != nullptr) {
        const float d0 = (float)(k0 - row);
#pragma unroll
        for (int i = 0; i < 128; ++i)
          s[i] = __float_as_uint(fmaf(alibi_s, d0 + (float)i, __uint_as_float(s[i])));   // -inf stays -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(s[i]));
        mx1 = fmaxf(mx1, __uint_as_float(s[i + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(s[i + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(s[i + 3]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;
      const float m_new = fmaxf(m_used, mx);
      const bool grow = (m_new - m_used) > kFaRescaleThreshold;
      float alpha = 1.f;
      if (grow) {
        alpha = exp2f(m_used - m_new);
        m_used = m_new;
        l *= alpha;
      }
      // P(j) overwrites the tile PV(j-1) reads, and a rescale touches O: wait for PV(j-1) (issued a whole
      // softmax period ago, so this rarely blocks)
      if (threadIdx.x == 64) FA_TRACE(1, j, 3);
      if (j > 0 && !mbar_wait(&sh->pv_done[t], (j - 1) & 1, abort_flag)) fail();
      if (threadIdx.x == 64) FA_TRACE(1, j, 4);
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_o + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32(t_o + c * 32, v);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      // P = exp2(s*scale - m_used) -> bf16 -> swizzled smem, 8 columns (one 16-byte chunk) at a time
      float ps0 = 0.f, ps1 = 0.f, ps2 = 0.f, ps3 = 0.f;
      const float neg_m = -m_used;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) p[i] = exp2f(fmaf(__uint_as_float(s[c * 8 + i]), scale_log2, neg_m));
        ps0 += p[0] + p[4]; ps1 += p[1] + p[5]; ps2 += p[2] + p[6]; ps3 += p[3] + p[7];
        *reinterpret_cast<bf16x8*>(p_row + (c >> 3) * (kFaTileBytes / 2) + (((c & 7) ^ sw) << 4)) = pack8(p);
      }
      l += (ps0 + ps1) + (ps2 + ps3);
      fence_proxy_async_smem();
      mbar_arrive(&sh->p_full[t]);
      if (threadIdx.x == 64) FA_TRACE(1, j, 5);
    }
    // ---------------- epilogue: O / l -> bf16 -> global; LSE ----------------
    if (my_n > 0) {
      if (!mbar_wait(&sh->pv_done[t], (my_n - 1) & 1, abort_flag)) fail();
      tc_fence_after();
      if (ok && !*abort_flag) {
        const float inv_l = row_valid ? 1.f / l : 0.f;
        __nv_bfloat16* orow = out + ((size_t)row * Hq + h) * kFaD;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_o + c * 32, v);
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
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // error path: give copies / MMAs still in flight time to land before smem and TMEM go away
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

#ifdef ELL_FA_TRACE
ELL_API int ell_flash_fwd_set_trace(long long* buf) {
  return (int)cudaMemcpyToSymbol(ell::g_fa_trace, &buf, sizeof(buf));
}
#endif

// Host-only: the forward kernel's plan for host-resident row_start [T], from the kernel's own arithmetic.  For every
// CTA tile pair p (query rows 256p ..) and tile t in {0, 1}: out[(2p + t) * 3 + {0, 1, 2}] = first key row, number of
// key tiles, and a bit mask (bit j set = key tile j is masked element-wise; only the first 31 tiles are recorded).
ELL_API int ell_flash_fwd_plan(const int* row_start, int T, int* out) {
  const int n_pairs = (T + 2 * kFaM - 1) / (2 * kFaM);
  for (int p = 0; p < n_pairs; ++p) {
    const int q0 = p * 2 * kFaM, kv_lo = row_start[q0];
    for (int t = 0; t < 2; ++t) {
      const int tile_first = q0 + t * kFaM;
      const int n = fa_num_kv_tiles(tile_first, T, kv_lo);
      const int last_row = (tile_first + kFaM < T ? tile_first + kFaM : T) - 1;
      const int max_row_start = n > 0 ? row_start[last_row] : 0;
      int bits = 0;
      for (int j = 0; j < n && j < 31; ++j)
        if (fa_tile_needs_mask(kv_lo + j * kFaN, tile_first, max_row_start)) bits |= 1 << j;
      int* o = out + (2 * p + t) * 3;
      o[0] = kv_lo;
      o[1] = n;
      o[2] = bits;
    }
  }
  return n_pairs;
}

// q [T, Hq, 128] / k, v [T, Hk, 128] bf16 with row strides (in elements) q_stride / kv_stride (views
// into the packed QKV GEMM output are fine); out [T, Hq, 128] contiguous; lse [Hq, T] fp32;
// row_start [T] int32 (document start of every token).  Causal.
// alibi_slopes: fp32 [Hq] or null.
ELL_API int ell_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* row_start,
                               int T, int Hq, int Hk, int q_stride, int kv_stride, float scale,
                               const float* alibi_slopes, int* err, cudaStream_t stream) {
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
  dim3 grid((T + 2 * kFaM - 1) / (2 * kFaM), Hq);
  flash_fwd_kernel<<<grid, kFaThreads, kFaSmemBytes, stream>>>(tq, tk, tv, (__nv_bfloat16*)out, lse, row_start, T, Hq,
                                                               Hk, scale * 1.4426950408889634f, alibi_slopes, err);
  return launch_status();
}
