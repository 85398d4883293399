// Causal flash attention backward on tcgen05 / TMEM for sm_100a: packed variable-length documents,
// MHA and GQA, head_dim 128, bf16 in/out, fp32 accumulation.
//
// One CTA per (128-key tile j, kv head); it walks the query tiles i >= j that can see those keys (and
// every query head of the kv head's group) and keeps dK_j, dV_j in TMEM for the whole walk:
//   S  = Q_i K_j^T            P  = exp2(S*scale*log2e - lse_i*log2e)        (causal / document mask)
//   dP = dO_i V_j^T           dS = P * (dP - delta_i) * scale               delta = rowsum(dO * O)
//   dV_j += P^T dO_i          dK_j += dS^T Q_i          dQ_i += dS K_j      (fp32, reduced across CTAs)
// 320 threads:
//   warp 0      TMA: K_j, V_j once; Q_i, dO_i per step
//   warp 1      one thread issues the five MMAs of a step; TMEM columns: S 0-127, dP|dQ 128-255,
//               dV 256-383, dK 384-511.  P and dS reach the tensor core through swizzled shared memory;
//               the transposed operands (P^T, dS^T, and dO, Q, K as [k x n] operands) are read in place
//               with MN-major descriptors, so nothing is transposed in memory.
//   warps 2-9   two groups of 128 threads; thread r of a group owns query row r (TMEM lane r) and half of
//               the 128 columns.  They turn S into P and dP into dS, drain the dQ tile (TMEM -> swizzled
//               fp32 staging, half in the dS buffer and half in a dedicated tile -> cp.reduce.async.bulk add
//               into the fp32 dQ accumulator; nothing waits for the adds until the buffers are needed again),
//               and at the end write dV_j / dK_j.
// Order of a step: S_i is issued as soon as Q_i has landed (its columns were read out a step ago), dP_i after the dQ
// tile of step i-1 has been drained from the columns they share (dP is not needed before the P pass is over), dQ_i
// before dK_i, so the drain of dQ_i overlaps dK_i: the softmax warps never wait for an MMA that could have run earlier.
// Every wait is bounded; on expiry the CTA records an error code, runs the remaining steps without
// touching global memory, frees its TMEM and returns.
//
// Backward of flash_attn_varlen_{qkv,kv}packed_func used by the reference
// (llm/models/mg_models/llama/transformer.py:65-143).
#include "common.cuh"
#include "sm100.cuh"

namespace ell {
using namespace sm100;

constexpr int kFbThreads = 320;
constexpr int kFbTile = 128, kFbD = 128;
constexpr int kFbSfuGroup = 0;    // of every four 8-column groups this one keeps ex2 on the special-function unit (measured: none is slower)
constexpr int kFbTileBytes = 128 * 128 * 2;   // 32 KiB
constexpr int kFbHalf = kFbTileBytes / 2;     // 16 KiB: one 64-column half of a tile
constexpr int kFbSmemBytes = 7 * kFbTileBytes + 1024 + 256;   // K, V, Q, dO, P, dS, dQ staging

struct FbShared {
  uint64_t kv_full, q_full, do_full, q_empty, do_empty, s_full, dp_full, p_full, ds_full, dq_full, dq_drained;
  uint32_t tmem_base;
  int abort_flag;
};

enum FbErr { kFbErrProducer = 21, kFbErrMma = 22, kFbErrSoftmax = 23 };

// Optional timeline of the first CTA (clock64 stamps per role, step and stage), compiled in with -DELL_FA_TRACE.
#ifdef ELL_FA_TRACE
__device__ long long* g_fb_trace = nullptr;   // [3 roles][64 steps][8 stages]
#define FB_TRACE(role, it, slot)                                                             \
  do {                                                                                       \
    if (blockIdx.x == 0 && blockIdx.y == 0 && g_fb_trace && (it) < 64)                       \
      g_fb_trace[(((role) * 64 + (it)) << 3) + (slot)] = clock64();                          \
  } while (0)
#else
#define FB_TRACE(role, it, slot)
#endif

// Index one past the last query tile that can see keys up to k_last: row_start is non-decreasing, so the
// tiles whose first row starts a document after k_last (and all later tiles) are invisible.  Warp-uniform.
__device__ __forceinline__ int fb_last_qtile(const int* __restrict__ row_start, int j, int n_qt, int k_last, int lane) {
  int i_end = j + 1;
  for (int base = j + 1; base < n_qt; base += 32) {
    const int i = base + lane;
    const bool vis = i < n_qt && row_start[i * kFbTile] <= k_last;
    const unsigned m = __ballot_sync(0xffffffffu, vis);
    i_end = base + __popc(m);
    if (m != 0xffffffffu) break;
  }
  return i_end;
}

// registers are granted per 4 warps: 10 warps count as 12, which caps a thread at 168 registers
__global__ void __launch_bounds__(kFbThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                 const __grid_constant__ CUtensorMap tmDQ, const float* __restrict__ lse,
                 const float* __restrict__ delta, const int* __restrict__ row_start,
                 __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, int dkv_stride,
                 float* __restrict__ dkv_acc, int nsplit, int T, int Hq, int Hk, float scale,
                 const float* __restrict__ alibi_slopes, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + 1 * kFbTileBytes;
  uint8_t* sQ = smem + 2 * kFbTileBytes;
  uint8_t* sdO = smem + 3 * kFbTileBytes;
  uint8_t* sP = smem + 4 * kFbTileBytes;
  uint8_t* sdS = smem + 5 * kFbTileBytes;
  uint8_t* sStage = smem + 6 * kFbTileBytes;   // fp32 staging of half of each dQ tile (the other half reuses dS)
  FbShared* sh = reinterpret_cast<FbShared*>(smem + 7 * kFbTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (T + kFbTile - 1) / kFbTile;
  // blockIdx.y = key tile (j = 0 has the longest walk; with x varying fastest the heaviest CTAs of every head
  // are scheduled first), blockIdx.x = kv head x split of its query-head group.
  const int j = blockIdx.y;
  const int kvh = blockIdx.x / nsplit;
  const int G = Hq / Hk / nsplit;              // query heads walked by this CTA
  const int h_first = kvh * (Hq / Hk) + (blockIdx.x % nsplit) * G;
  const int k0 = j * kFbTile;
  const int k_last = min(k0 + kFbTile, T) - 1;
  const int i_end = fb_last_qtile(row_start, j, n_qt, k_last, lane);
  const int n_it = G * (i_end - j);

  if (threadIdx.x == 0) {
    mbar_init(&sh->kv_full, 1);
    mbar_init(&sh->q_full, 1);
    mbar_init(&sh->q_empty, 1);
    mbar_init(&sh->do_full, 1);
    mbar_init(&sh->do_empty, 1);
    mbar_init(&sh->s_full, 1);
    mbar_init(&sh->dp_full, 1);
    mbar_init(&sh->p_full, 256);
    mbar_init(&sh->ds_full, 256);
    mbar_init(&sh->dq_full, 1);
    mbar_init(&sh->dq_drained, 256);
    sh->abort_flag = *(volatile int*)err;   // an earlier CTA already failed: do not wait on anything
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
    tma_prefetch_desc(&tmDQ);
  }
  if (warp == 1) tmem_alloc<512>(&sh->tmem_base);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const bool dead_on_arrival = sh->abort_flag != 0;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 384;
  volatile int* abort_flag = &sh->abort_flag;

  if (dead_on_arrival) {
    // fall through to the common exit: nothing was issued
  } else if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(&sh->kv_full, 2 * kFbTileBytes);
      tma_load_2d(sK, &tmK, &sh->kv_full, kvh * kFbD, k0);
      tma_load_2d(sK + kFbHalf, &tmK, &sh->kv_full, kvh * kFbD + 64, k0);
      tma_load_2d(sV, &tmV, &sh->kv_full, kvh * kFbD, k0);
      tma_load_2d(sV + kFbHalf, &tmV, &sh->kv_full, kvh * kFbD + 64, k0);
      int it = 0;
      for (int g = 0; g < G && ok; ++g) {
        const int h = h_first + g;
        for (int i = j; i < i_end; ++i, ++it) {
          // dO is released by the dV MMA (mid-step), Q by the dK MMA (end of step): the next tiles
          // stream in while the current step computes dS and drains dQ
          FB_TRACE(2, it, 0);
          if (it > 0 && !mbar_wait(&sh->do_empty, (it - 1) & 1, abort_flag)) { ok = false; break; }
          FB_TRACE(2, it, 1);
          mbar_expect_tx(&sh->do_full, kFbTileBytes);
          tma_load_2d(sdO, &tmdO, &sh->do_full, h * kFbD, i * kFbTile);
          tma_load_2d(sdO + kFbHalf, &tmdO, &sh->do_full, h * kFbD + 64, i * kFbTile);
          if (it > 0 && !mbar_wait(&sh->q_empty, (it - 1) & 1, abort_flag)) { ok = false; break; }
          FB_TRACE(2, it, 2);
          mbar_expect_tx(&sh->q_full, kFbTileBytes);
          tma_load_2d(sQ, &tmQ, &sh->q_full, h * kFbD, i * kFbTile);
          tma_load_2d(sQ + kFbHalf, &tmQ, &sh->q_full, h * kFbD + 64, i * kFbTile);
        }
      }
      if (!ok) {
        sh->abort_flag = 1;
        atomicCAS(err, 0, kFbErrProducer);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(128, 128, false, false);  // A, B K-major
      constexpr uint32_t idesc_mm = make_idesc_bf16(128, 128, true, true);    // A, B MN-major
      constexpr uint32_t idesc_km = make_idesc_bf16(128, 128, false, true);   // A K-major, B MN-major
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_addr = smem_u32(sQ), do_addr = smem_u32(sdO);
      const uint32_t p_addr = smem_u32(sP), ds_addr = smem_u32(sdS);
      bool ok = mbar_wait(&sh->kv_full, 0, abort_flag);
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t ph = it & 1;
        FB_TRACE(0, it, 0);
        // S = Q K^T: its columns were read out by the P pass of the previous step long ago
        if (!mbar_wait(&sh->q_full, ph, abort_flag)) { ok = false; break; }
        FB_TRACE(0, it, 1);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kFbHalf + (k & 3) * 32;
          umma_bf16(t_s, make_smem_desc(q_addr + off, 16, 1024), make_smem_desc(k_addr + off, 16, 1024), idesc_kk,
                    k != 0);
        }
        umma_commit(&sh->s_full);
        // dP = dO V^T into the columns the previous dQ tile is drained from (dP is not needed before the P pass is over)
        if (!mbar_wait(&sh->do_full, ph, abort_flag)) { ok = false; break; }
        if (it > 0 && !mbar_wait(&sh->dq_drained, (it - 1) & 1, abort_flag)) { ok = false; break; }
        FB_TRACE(0, it, 2);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kFbHalf + (k & 3) * 32;
          umma_bf16(t_dp, make_smem_desc(do_addr + off, 16, 1024), make_smem_desc(v_addr + off, 16, 1024), idesc_kk,
                    k != 0);
        }
        umma_commit(&sh->dp_full);
        // dV += P^T dO
        if (!mbar_wait(&sh->p_full, ph, abort_flag)) { ok = false; break; }
        FB_TRACE(0, it, 3);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(t_dv, make_smem_desc(p_addr + k * 2048, kFbHalf, 1024),
                    make_smem_desc(do_addr + k * 2048, kFbHalf, 1024), idesc_mm, (it | k) != 0);
        umma_commit(&sh->do_empty);
        // dQ = dS K first (into the dP columns, which the dS pass has read out): the softmax warps start draining it
        // while dK += dS^T Q still runs
        if (!mbar_wait(&sh->ds_full, ph, abort_flag)) { ok = false; break; }
        FB_TRACE(0, it, 4);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kFbHalf + (k & 3) * 32;
          umma_bf16(t_dp, make_smem_desc(ds_addr + off, 16, 1024), make_smem_desc(k_addr + k * 2048, kFbHalf, 1024),
                    idesc_km, k != 0);
        }
        umma_commit(&sh->dq_full);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(t_dk, make_smem_desc(ds_addr + k * 2048, kFbHalf, 1024),
                    make_smem_desc(q_addr + k * 2048, kFbHalf, 1024), idesc_mm, (it | k) != 0);
        umma_commit(&sh->q_empty);     // also: dV, dK of this step done; P, dS, Q free
        FB_TRACE(0, it, 5);
      }
      if (!ok) {
        sh->abort_flag = 1;
        atomicCAS(err, 0, kFbErrMma);
      }
    }
  } else {
    // ------------------- softmax / dS / dQ drain / epilogue: thread <-> row -------------------
    const int wg = (warp - 2) >> 2;              // column half: 0 -> columns 0-63, 1 -> 64-127
    const int quad = warp & 3;                   // TMEM lane quadrant this warp may access
    const int r = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const int col_base = wg * 64;
    const float scale_log2 = scale * 1.4426950408889634f;
    uint8_t* p_row = sP + wg * kFbHalf + r * 128;     // this thread's 128-byte row in its half of P / dS
    uint8_t* ds_row = sdS + wg * kFbHalf + r * 128;
    const int sw = r & 7;
    bool ok = true;
    auto fail = [&]() {
      ok = false;
      sh->abort_flag = 1;
      atomicCAS(err, 0, kFbErrSoftmax);
    };
    int it = 0;
    for (int g = 0; g < G; ++g) {
      const int h = h_first + g;
      for (int i = j; i < i_end; ++i, ++it) {
        const uint32_t ph = it & 1;
        const int q0 = i * kFbTile;
        const int row = q0 + r;
        const bool row_valid = row < T;
        const int my_start = row_valid ? row_start[row] : 0x7fffffff;
        const float lse2 = row_valid ? lse[(size_t)h * T + row] * 1.4426950408889634f : 0.f;
        const float dlt = row_valid ? delta[(size_t)h * T + row] : 0.f;
        // ALiBi: P is recomputed with the forward's bias slope * (key - query) (a constant of q and k: no gradient)
        const float slope2 = alibi_slopes != nullptr ? alibi_slopes[h] * 1.4426950408889634f : 0.f;
        const bool need_mask = (i == j) || (row_start[min(q0 + kFbTile, T) - 1] > k0) || (q0 + kFbTile > T);
        uint32_t pk[32];                         // P of this thread's 64 columns, packed bf16x2
        if (threadIdx.x == 64) FB_TRACE(1, it, 0);
        if (!mbar_wait(&sh->s_full, ph, abort_flag)) fail();
        if (threadIdx.x == 64) FB_TRACE(1, it, 1);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_s + lane_off + col_base + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            // exp2(s * scale - lse): the exponentials and the two bf16 conversions of a score share the 4-lane
            // special-function pipe; three of every four 8-column groups use the FMA-pipe polynomial instead
            float p[8];
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
              float off0 = -lse2, off1 = -lse2;
              if (alibi_slopes != nullptr) {
                const float d0 = (float)(k0 + col_base + c * 32 + g8 * 8 + e - row);
                off0 = fmaf(slope2, d0, -lse2);
                off1 = fmaf(slope2, d0 + 1.f, -lse2);
              }
              const float2 x = ffma2(make_float2(__uint_as_float(v[g8 * 8 + e]), __uint_as_float(v[g8 * 8 + e + 1])),
                                     make_float2(scale_log2, scale_log2), make_float2(off0, off1));
              float2 pe;
              if (g8 != kFbSfuGroup) {
                pe = exp2_poly2(x);
              } else {
                pe.x = ex2_approx(x.x);
                pe.y = ex2_approx(x.y);
              }
              p[e] = pe.x;
              p[e + 1] = pe.y;
            }
            if (need_mask) {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const int kidx = k0 + col_base + c * 32 + g8 * 8 + e;
                if (kidx > row || kidx < my_start || !row_valid) p[e] = 0.f;
              }
            }
            bf16x8 b = pack8(p);
            *reinterpret_cast<bf16x8*>(p_row + (((c * 4 + g8) ^ sw) << 4)) = b;
#pragma unroll
            for (int e = 0; e < 4; ++e) pk[c * 16 + g8 * 4 + e] = *reinterpret_cast<uint32_t*>(&b.v[e]);
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(&sh->p_full);
        if (threadIdx.x == 64) FB_TRACE(1, it, 2);
        if (!mbar_wait(&sh->dp_full, ph, abort_flag)) fail();
        if (threadIdx.x == 64) FB_TRACE(1, it, 3);
        tc_fence_after();
        if (it > 0) {
          // half of the previous dQ tile was staged in this group's half of the dS buffer (the older of the
          // two reduce-add groups): it must have been read before dS overwrites it
          if (r == 0) tma_store_wait_read<1>();
          named_bar_sync(1 + wg, 128);
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_dp + lane_off + col_base + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            // dS = P * (dP - delta) * scale, two scores per instruction: (dP * scale - delta * scale), then times P
            float d[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 pp = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&pk[c * 16 + g8 * 4 + e]));
              const float2 t = ffma2(make_float2(__uint_as_float(v[g8 * 8 + 2 * e]), __uint_as_float(v[g8 * 8 + 2 * e + 1])),
                                     make_float2(scale, scale), make_float2(-dlt * scale, -dlt * scale));
              const float2 ds = ffma2(pp, t, make_float2(0.f, 0.f));
              d[2 * e] = ds.x;
              d[2 * e + 1] = ds.y;
            }
            *reinterpret_cast<bf16x8*>(ds_row + (((c * 4 + g8) ^ sw) << 4)) = pack8(d);
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(&sh->ds_full);
        if (threadIdx.x == 64) FB_TRACE(1, it, 4);
        // ---- dQ tile: TMEM -> fp32 staging (this group's halves of the P and dS buffers) -> reduce-add
        if (!mbar_wait(&sh->dq_full, ph, abort_flag)) fail();
        if (threadIdx.x == 64) FB_TRACE(1, it, 5);
        tc_fence_after();
        if (it > 0) {
          // the dedicated staging half was last read by the newer reduce-add group of the previous step
          if (r == 0) tma_store_wait_read<0>();
          named_bar_sync(1 + wg, 128);
        }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = 1 - cc;                  // the half staged in the dedicated tile first
          // the other half goes into this group's half of the dS buffer, which dK (issued after dQ) reads until q_empty
          if (c == 0 && !mbar_wait(&sh->q_empty, ph, abort_flag)) fail();
          uint32_t v[32];
          tmem_ld_32x32(t_dp + lane_off + col_base + c * 32, v);
          tmem_ld_wait();
          uint8_t* st_row = (c == 0 ? sdS : sStage) + wg * kFbHalf + r * 128;
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4)
            *reinterpret_cast<uint4*>(st_row + ((g4 ^ sw) << 4)) =
                make_uint4(v[g4 * 4], v[g4 * 4 + 1], v[g4 * 4 + 2], v[g4 * 4 + 3]);
        }
        tc_fence_before();
        mbar_arrive(&sh->dq_drained);
        fence_proxy_async_smem();
        named_bar_sync(1 + wg, 128);
        if (r == 0) {
          if (!*abort_flag) {
            tma_reduce_add_2d(&tmDQ, sdS + wg * kFbHalf, h * kFbD + col_base, q0);
            tma_store_commit();            // older group: the dS buffer is needed again first
            tma_reduce_add_2d(&tmDQ, sStage + wg * kFbHalf, h * kFbD + col_base + 32, q0);
            tma_store_commit();
          }
        }
        if (threadIdx.x == 64) FB_TRACE(1, it, 6);
      }
    }
    // ---------------- epilogue: dV (group 0) / dK (group 1) -> bf16 -> global ----------------
    // Every step's drain waited for q_empty, which is committed after dK (and so after dV) of that step.
    if (n_it > 0 && ok && !*abort_flag && nsplit > 1) {
      // the query-head group is split over CTAs: add into the fp32 accumulators [2][T, Hk*128] (dk, dv)
      const int key = k0 + r;
      const uint32_t t_acc = (wg == 0 ? t_dv : t_dk) + lane_off;
      float* dst = dkv_acc + (wg == 0 ? (size_t)T * Hk * kFbD : 0) + ((size_t)key * Hk + kvh) * kFbD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_acc + c * 32, v);
        tmem_ld_wait();
        if (key < T) {
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4)
            atomicAdd(reinterpret_cast<float4*>(dst + c * 32 + g4 * 4),
                      make_float4(__uint_as_float(v[g4 * 4]), __uint_as_float(v[g4 * 4 + 1]),
                                  __uint_as_float(v[g4 * 4 + 2]), __uint_as_float(v[g4 * 4 + 3])));
        }
      }
    } else if (n_it > 0 && ok && !*abort_flag) {
      const int key = k0 + r;
      const uint32_t t_acc = (wg == 0 ? t_dv : t_dk) + lane_off;
      __nv_bfloat16* dst = (wg == 0 ? dv : dk) + (size_t)key * dkv_stride + (size_t)kvh * kFbD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_acc + c * 32, v);
        tmem_ld_wait();
        if (key < T) {
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[g8 * 8 + e]);
            *reinterpret_cast<bf16x8*>(dst + c * 32 + g8 * 8) = pack8(f);
          }
        }
      }
    }
    if (r == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<512>(tmem_base);
  }
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h).
__global__ void flash_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                       float* __restrict__ delta, int T, int Hq) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= T * Hq) return;
  const int t = w / Hq, h = w % Hq;
  const uint2 a = reinterpret_cast<const uint2*>(o + (size_t)w * kFbD)[lane];
  const uint2 b = reinterpret_cast<const uint2*>(dout + (size_t)w * kFbD)[lane];
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
  const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  s = warp_sum(s);
  if (lane == 0) delta[(size_t)h * T + t] = s;
}

// dq (bf16, row stride dq_stride elements) = dq_acc (fp32 [T, W]); 8 elements per thread.
__global__ void flash_bwd_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int T, int W,
                                            int dq_stride) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int vec_per_row = W / 8;
  if (idx >= (size_t)T * vec_per_row) return;
  const int t = idx / vec_per_row, c = idx % vec_per_row;
  const float4 x = reinterpret_cast<const float4*>(acc + (size_t)t * W)[2 * c];
  const float4 y = reinterpret_cast<const float4*>(acc + (size_t)t * W)[2 * c + 1];
  const float f[8] = {x.x, x.y, x.z, x.w, y.x, y.y, y.z, y.w};
  reinterpret_cast<bf16x8*>(dq + (size_t)t * dq_stride)[c] = pack8(f);
}

int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                      uint32_t box_inner, uint32_t box_outer);
int make_tmap_f32_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                     uint32_t box_inner, uint32_t box_outer);

}  // namespace ell

using namespace ell;

#ifdef ELL_FA_TRACE
ELL_API int ell_flash_bwd_set_trace(long long* buf) {
  return (int)cudaMemcpyToSymbol(ell::g_fb_trace, &buf, sizeof(buf));
}
#endif

// q [T, Hq, 128], k / v [T, Hk, 128] (row strides q_stride / kv_stride elements, views into a packed QKV
// buffer are fine); out, dout [T, Hq, 128] contiguous; lse [Hq, T] from the forward.
// Outputs: dq [T, Hq, 128] (row stride dq_stride), dk / dv [T, Hk, 128] (row stride dkv_stride) - views into
// one packed dQKV buffer are fine.  Scratch: dq_acc fp32 [T, Hq*128] (zeroed here), delta fp32 [Hq, T],
// dkv_acc fp32 [2, T, Hk*128] (GQA only, may be null: used when the head group is split over CTAs).
ELL_API int ell_flash_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                               const float* lse, const int* row_start, void* dq, void* dk, void* dv, float* dq_acc,
                               float* delta, float* dkv_acc, int T, int Hq, int Hk, int q_stride, int kv_stride, int dq_stride,
                               int dkv_stride, float scale, const float* alibi_slopes, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (Hq % Hk) return -2;
  if ((dq_stride % 8) || (dkv_stride % 8)) return -3;
  CUtensorMap tq, tk, tv, tdo, tdq;
  int rc = make_tmap_bf16_2d(&tq, q, (uint64_t)Hq * kFbD, (uint64_t)T, (uint64_t)q_stride * 2, 64, 128);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tk, k, (uint64_t)Hk * kFbD, (uint64_t)T, (uint64_t)kv_stride * 2, 64, 128);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tv, v, (uint64_t)Hk * kFbD, (uint64_t)T, (uint64_t)kv_stride * 2, 64, 128);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tdo, dout, (uint64_t)Hq * kFbD, (uint64_t)T, (uint64_t)Hq * kFbD * 2, 64, 128);
  if (rc) return rc;
  rc = make_tmap_f32_2d(&tdq, dq_acc, (uint64_t)Hq * kFbD, (uint64_t)T, (uint64_t)Hq * kFbD * 4, 32, 128);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFbSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int W = Hq * kFbD;
  const int n_kt = (T + kFbTile - 1) / kFbTile;
  // few kv heads and a short sequence leave SMs idle: split each query-head group over CTAs
  const int nsplit = (Hq > Hk && dkv_acc != nullptr && Hk * n_kt < 2 * kNumSMs) ? Hq / Hk : 1;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, (size_t)T * W * sizeof(float), stream);
  if (e != cudaSuccess) return (int)e;
  if (nsplit > 1) {
    e = cudaMemsetAsync(dkv_acc, 0, (size_t)2 * T * Hk * kFbD * sizeof(float), stream);
    if (e != cudaSuccess) return (int)e;
  }
  {
    const long long warps = (long long)T * Hq;
    const int threads = 256;
    const unsigned blocks = (unsigned)((warps * 32 + threads - 1) / threads);
    flash_bwd_delta_kernel<<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, delta,
                                                           T, Hq);
  }
  dim3 grid(Hk * nsplit, n_kt);
  flash_bwd_kernel<<<grid, kFbThreads, kFbSmemBytes, stream>>>(tq, tk, tv, tdo, tdq, lse, delta, row_start,
                                                               (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, dkv_stride,
                                                               dkv_acc, nsplit, T, Hq, Hk, scale, alibi_slopes, err);
  if (nsplit > 1) {
    const int Wk = Hk * kFbD;
    const size_t n = (size_t)T * (Wk / 8);
    flash_bwd_dq_convert_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(dkv_acc, (__nv_bfloat16*)dk, T, Wk,
                                                                                 dkv_stride);
    flash_bwd_dq_convert_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(dkv_acc + (size_t)T * Wk,
                                                                                 (__nv_bfloat16*)dv, T, Wk, dkv_stride);
  }
  {
    const size_t n = (size_t)T * (W / 8);
    flash_bwd_dq_convert_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(dq_acc, (__nv_bfloat16*)dq, T, W,
                                                                                 dq_stride);
  }
  return launch_status();
}
