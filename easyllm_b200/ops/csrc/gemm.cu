// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM), sm_100a.
//
//   C[M,N] (+)= op(A)[M,K] · op(B)[N,K]^T        bf16 in, fp32 accumulate
//
// Operand storage: "K-major" A is row-major [M,K] (the reduction dim is contiguous), "MN-major"
// A is row-major [K,M]; the same for B with N.  The three GEMMs of a linear layer map to
//   forward  y  = x · Wᵀ      A = x  (K-major)   B = W  (K-major)
//   dgrad    dx = dy · W      A = dy (K-major)   B = W  (MN-major: stored [N_red, K_out])
//   wgrad    dW = dyᵀ · x     A = dy (MN-major)  B = x  (MN-major), fp32 accumulate into the
//                                                 flat gradient buffer (beta = 1)
// so no transposed copy of an activation or weight is ever materialised.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D tiles (128B swizzle) into a 4–6 stage ring
//   warp 1      allocates TMEM, one thread issues tcgen05.mma (128 x BN x 16 per instruction),
//               tcgen05.commit releases smem stages and publishes finished accumulators
//   warps 2-5   epilogue: tcgen05.ld TMEM -> registers -> (bias) -> bf16 -> swizzled smem ->
//               TMA store, or fp32 read-modify-write to global for gradient accumulation
// Two accumulators (2 x BN TMEM columns) let the epilogue of tile i overlap the main loop of
// tile i+1.  Tiles are walked M-fastest so CTAs running together share the B (weight) tile in L2.
//
// This replaces the cuBLAS calls behind torch.matmul / F.linear in the reference
// (llm/models/mg_models/base_modules/layers/column_parallel_linear.py:42,68,99,
//  row_parallel_linear.py:113, llama/lm_head.py:62-66).
#include "gemm_fuse.cuh"

namespace ell {

constexpr int kABytes = kBM * kBK * 2;     // 16 KiB
constexpr int kGroupM = 16;   // tiles are walked in groups of 16 M-tiles x all N-tiles for L2 reuse

// The tile-order functions below are __host__ __device__: ell_gemm_enumerate_units runs the very same code on the
// host so a CPU test can check that every launch covers each output tile exactly once, in the intended order.
__host__ __device__ __forceinline__ void swizzle_tile(int idx, int tiles_m, int tiles_n, int& mt, int& nt) {
  const int width = kGroupM * tiles_n;
  const int group = idx / width, rem = idx % width;
  const int first_m = group * kGroupM;
  const int gsz = (tiles_m - first_m) < kGroupM ? (tiles_m - first_m) : kGroupM;
  mt = first_m + rem % gsz;
  nt = rem / gsz;
}

template <int FUSE>
__host__ __device__ __forceinline__ void map_tile(int idx, int tiles_m, int tiles_n, const FuseArgs& f, int& mt, int& nt) {
  if (FUSE == kFuseAG) {
    const int tpr = tiles_m / f.tp, per_phase = tpr * tiles_n;
    const int phase = idx / per_phase;
    int mi;
    swizzle_tile(idx % per_phase, tpr, tiles_n, mi, nt);
    mt = ((f.rank + phase) % f.tp) * tpr + mi;
  } else if (FUSE == kFuseRS || FUSE == kFuseAR) {
    int mp;
    swizzle_tile(idx, tiles_m, tiles_n, mp, nt);
    mt = (mp % f.tp) * (tiles_m / f.tp) + mp / f.tp;   // interleave owners so every owner is fed evenly
  } else {
    swizzle_tile(idx, tiles_m, tiles_n, mt, nt);
  }
}

// Work units of a plain (unfused) launch.  When the last wave would leave more than half of the CTAs idle,
// each of its tiles is cut into two half-width tiles (BN/2 columns), so the tail costs half a wave:
// units [0, num_full) are whole tiles, unit num_full + 2i + h is half h of tile num_full + i.
struct TileUnit {
  int mt, nt, n0, bn;
};

__host__ __device__ inline int split_tail_tiles(int num_tiles, int ctas, bool allowed) {
  const int tail = num_tiles % ctas;
  return (allowed && tail > 0 && 2 * tail <= ctas) ? tail : 0;
}

template <int BN, int FUSE>
__host__ __device__ __forceinline__ TileUnit decode_unit(int unit, int tiles_m, int tiles_n, int num_full, const FuseArgs& f) {
  TileUnit u;
  int tile = unit, half = -1;
  if (FUSE == kFuseNone && unit >= num_full) {
    tile = num_full + ((unit - num_full) >> 1);
    half = (unit - num_full) & 1;
  }
  map_tile<FUSE>(tile, tiles_m, tiles_n, f, u.mt, u.nt);
  u.bn = half >= 0 ? BN / 2 : BN;
  u.n0 = u.nt * BN + (half > 0 ? BN / 2 : 0);
  return u;
}

template <int BN>
struct GemmCfg {
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 2 * kEpiBufBytes + 1024 /*align slack*/ + 256;
};

struct GemmShared {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int epi_abort;
};

template <int BN, bool A_MN, bool B_MN, int OUT, bool HAS_BIAS, int FUSE>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmA2,
                 const __grid_constant__ FuseArgs fuse,
                 const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc, int* __restrict__ err) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + Cfg::kStages * kABytes;
  uint8_t* sC = smem + Cfg::kStages * Cfg::kStageBytes;
  GemmShared* sh = reinterpret_cast<GemmShared*>(sC + 2 * kEpiBufBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + kBK - 1) / kBK;
  const int n_comm = FUSE == kFuseNone ? 0 : fuse.n_comm;
  const int cta0 = (int)blockIdx.x - n_comm;            // index among the GEMM CTAs
  const int cta_stride = (int)gridDim.x - n_comm;
  const int n_split = split_tail_tiles(num_tiles, cta_stride, FUSE == kFuseNone && BN == 256 && OUT != kOutBf16CE &&
                                                               !fuse.no_tail_split);
  const int num_full = num_tiles - n_split;
  const int num_units = num_tiles + n_split;

  if (FUSE != kFuseNone && (int)blockIdx.x < n_comm) {
    if (FUSE == kFuseAG) ag_comm_role(fuse, K, err, smem, 0, n_comm);
    else rs_reduce_role<BN>(fuse, N, tiles_n, err, smem, (int)gridDim.x, false, FUSE == kFuseAR);
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sh->tmem_full[a], 1);
      mbar_init(&sh->tmem_empty[a], kEpiThreads);
    }
    sh->abort_flag = 0;
    sh->epi_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) tmem_alloc<Cfg::kTmemCols>(&sh->tmem_base);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cta0; tile < num_units && ok; tile += cta_stride) {
        const TileUnit u = decode_unit<BN, FUSE>(tile, tiles_m, tiles_n, num_full, fuse);
        const int mt = u.mt, m0 = mt * kBM, n0 = u.n0;
        // half-width units load B through the second map (box of BN/2 rows; plain launches only)
        const CUtensorMap* b_map = (FUSE == kFuseNone && u.bn != BN) ? &tmA2 : &tmB;
        const uint32_t stage_bytes = kABytes + (uint32_t)u.bn * kBK * 2;
        const CUtensorMap* a_map = &tmA;
        int a_row = m0;
        if (FUSE == kFuseAG) {
          // rows of this tile come from rank `src`: the local shard is read in place, a remote shard
          // from the local gathered buffer once the peer's copy of this tile is flagged
          const int src = m0 / fuse.rows_per_rank;
          if (src == fuse.rank) {
            a_map = &tmA2;
            a_row = m0 - src * fuse.rows_per_rank;
          } else {
            const uint32_t* fl = fuse.flag_ptrs[fuse.rank] + (size_t)src * fuse.flags_per_src +
                                 (m0 - src * fuse.rows_per_rank) / kBM;
            if (!wait_flag_ge(fl, fuse.epoch, abort_flag)) {
              ok = false;
              atomicCAS(err, 0, kErrFlagWait);
              break;
            }
            fence_proxy_async_all();   // peer writes -> TMA reads (async proxy)
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&sh->full[stage], stage_bytes);
          uint8_t* a_dst = sA + stage * kABytes;
          uint8_t* b_dst = sB + stage * Cfg::kBBytes;
          if (!A_MN) {
            tma_load_2d(a_dst, a_map, &sh->full[stage], kb * kBK, a_row);
          } else {
#pragma unroll
            for (int i = 0; i < kBM / 64; ++i)
              tma_load_2d(a_dst + i * (64 * kBK * 2), &tmA, &sh->full[stage], m0 + i * 64, kb * kBK);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, b_map, &sh->full[stage], kb * kBK, n0);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              if (i * 64 < u.bn) tma_load_2d(b_dst + i * (64 * kBK * 2), &tmB, &sh->full[stage], n0 + i * 64, kb * kBK);
          }
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        sh->abort_flag = 1;
        atomicCAS(err, 0, kErrProducer);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_full = make_idesc_bf16(kBM, BN, A_MN, B_MN);
      constexpr uint32_t idesc_half = make_idesc_bf16(kBM, BN / 2, A_MN, B_MN);
      // K-major: 8-row groups 1024 B apart; one K=16 step is 32 B inside the swizzle row.
      // MN-major: 64-element MN groups one [64 x kBK] box (8 KiB) apart, 8-K groups 1024 B apart;
      // one K=16 step is two such groups (2 KiB).
      constexpr uint32_t a_lbo = A_MN ? 64 * kBK * 2 : 16, a_sbo = 1024, a_kstep = A_MN ? 2048 : 32;
      constexpr uint32_t b_lbo = B_MN ? 64 * kBK * 2 : 16, b_sbo = 1024, b_kstep = B_MN ? 2048 : 32;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = cta0; tile < num_units && ok; tile += cta_stride, ++it) {
        const uint32_t idesc = (FUSE == kFuseNone && tile >= num_full) ? idesc_half : idesc_full;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&sh->tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * kABytes);
          const uint32_t b_addr = smem_u32(sB + stage * Cfg::kBBytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = make_smem_desc(a_addr + k * a_kstep, a_lbo, a_sbo);
            const uint64_t db = make_smem_desc(b_addr + k * b_kstep, b_lbo, b_sbo);
            umma_bf16(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma_commit(&sh->empty[stage]);
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&sh->tmem_full[acc]);
      }
      if (!ok) {
        sh->abort_flag = 1;
        atomicCAS(err, 0, kErrMma);
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    const bool leader = (threadIdx.x == 64);
    int it = 0;
    uint32_t store_count = 0;
    uint32_t* pending_flag = nullptr;   // RS: flag of the last staged tile, raised once its stores completed
    if ((FUSE == kFuseRS || FUSE == kFuseAR) && leader) {
      // peers must have finished reading last epoch's staged tiles before they are overwritten
      for (int p = 0; p < fuse.tp; ++p)
        if (p != fuse.rank && !wait_flag_ge(fuse.done_ptrs[fuse.rank] + p, fuse.epoch - 1, abort_flag)) {
          sh->epi_abort = 1;
          atomicCAS(err, 0, kErrFlagWait);
        }
    }
    for (int tile = cta0; tile < num_units; tile += cta_stride, ++it) {
      const TileUnit u = decode_unit<BN, FUSE>(tile, tiles_m, tiles_n, num_full, fuse);
      const int mt = u.mt, nt = u.nt, m0 = mt * kBM, n0 = u.n0;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag)) sh->epi_abort = 1;
      named_bar_sync(1, kEpiThreads);
      if (*(volatile int*)&sh->epi_abort) break;   // uniform across the 128 epilogue threads
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      float ce_m = -INFINITY, ce_s = 0.f, ce_t = 0.f;
      int ce_tcol = -1;                          // target column inside this tile, if any
      if (OUT == kOutBf16CE) {
        const int row = m0 + row_in_tile;
        if (row < M) {
          const long long tc = fuse.ce_target[row] - fuse.ce_vocab_start - n0;
          if (tc >= 0 && tc < BN && tc + n0 < fuse.ce_valid) ce_tcol = (int)tc;
        }
      }
      if (OUT == kOutBf16 || OUT == kOutBf16CE) {
#pragma unroll 1
        for (int j = 0; j < u.bn / 64; ++j) {
          uint8_t* buf = sC + (store_count & 1) * kEpiBufBytes;
          if (leader) tma_store_wait_read<1>();
          named_bar_sync(1, kEpiThreads);
          uint32_t r[64];
          tmem_ld_32x32(t_row + j * 64, r);
          tmem_ld_32x32(t_row + j * 64 + 32, r + 32);
          tmem_ld_wait();
          if (HAS_BIAS) {
#pragma unroll
            for (int c = 0; c < 64; ++c) {
              const int col = n0 + j * 64 + c;
              const float b = col < N ? __bfloat162float(bias[col]) : 0.f;
              r[c] = __float_as_uint(__uint_as_float(r[c]) + b);
            }
          }
          if (OUT == kOutBf16CE) {
            // statistics of the logits as stored (rounded to bf16), so that backward's exp(logit - lse) sums to 1
            const int cbase = n0 + j * 64;
            float cm = -INFINITY;
#pragma unroll
            for (int c = 0; c < 64; ++c) {
              const float x = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[c])));
              r[c] = __float_as_uint(x);
              if (cbase + c < fuse.ce_valid) cm = fmaxf(cm, x);
              if (j * 64 + c == ce_tcol) ce_t = x;
            }
            if (cm > -INFINITY) {
              const float nm = fmaxf(ce_m, cm);
              float acc_s = ce_s * __expf(ce_m - nm);
#pragma unroll
              for (int c = 0; c < 64; ++c)
                if (cbase + c < fuse.ce_valid) acc_s += __expf(__uint_as_float(r[c]) - nm);
              ce_s = acc_s;
              ce_m = nm;
            }
          }
          uint8_t* row_ptr = buf + row_in_tile * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint4 v;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[c * 8 + 0]), __uint_as_float(r[c * 8 + 1]));
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[c * 8 + 2]), __uint_as_float(r[c * 8 + 3]));
            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[c * 8 + 4]), __uint_as_float(r[c * 8 + 5]));
            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[c * 8 + 6]), __uint_as_float(r[c * 8 + 7]));
            v.x = *reinterpret_cast<uint32_t*>(&p0);
            v.y = *reinterpret_cast<uint32_t*>(&p1);
            v.z = *reinterpret_cast<uint32_t*>(&p2);
            v.w = *reinterpret_cast<uint32_t*>(&p3);
            *reinterpret_cast<uint4*>(row_ptr + ((c ^ (row_in_tile & 7)) << 4)) = v;  // 128B swizzle
          }
          fence_proxy_async_smem();
          named_bar_sync(1, kEpiThreads);
          if (leader) {
            if (FUSE == kFuseRS || FUSE == kFuseAR) {
              const size_t off = stage_block<BN>(mt, nt, j, tiles_n);
              if (fuse_in_bounds(fuse, 0, off + kEpiBufBytes, err))
                bulk_store(reinterpret_cast<uint8_t*>(fuse.data_ptrs[fuse.rank]) + off, buf, kEpiBufBytes);
            } else if (n0 + j * 64 < N) {
              tma_store_2d(&tmC, buf, n0 + j * 64, m0);
            }
            tma_store_commit();
          }
          ++store_count;
        }
        if (OUT == kOutBf16CE) {
          const int row = m0 + row_in_tile;
          if (row < M) {
            float* part = fuse.ce_part + (size_t)nt * 3 * M + row;
            part[0] = ce_m;
            part[(size_t)M] = ce_s;
            part[(size_t)2 * M] = ce_t;
          }
        }
        if ((FUSE == kFuseRS || FUSE == kFuseAR) && leader) {
          // Publish the flag of the PREVIOUS tile: its bulk stores were committed BN/64 groups ago, so
          // waiting until at most BN/64 groups are pending does not stall behind this tile's stores.
          if (pending_flag != nullptr) {
            tma_store_wait_all<BN / 64>();
            fence_proxy_async_all();
            st_release_sys(pending_flag, fuse.epoch);
          }
          const int owner = m0 / fuse.rows_per_rank;
          const int mi = (m0 - owner * fuse.rows_per_rank) / kBM;
          pending_flag = fuse.flag_ptrs[owner] + (size_t)fuse.rank * fuse.flags_per_src + mi * tiles_n + nt;
        }
      } else {
        // fp32 output: 128 x 32 sub-tiles staged in swizzled smem, then a TMA store (overwrite) or
        // a TMA reduce-add (gradient accumulation: the add happens at L2, the SM never reads C)
#pragma unroll 1
        for (int j = 0; j < u.bn / 32; ++j) {
          uint8_t* buf = sC + (store_count & 1) * kEpiBufBytes;
          if (leader) tma_store_wait_read<1>();
          named_bar_sync(1, kEpiThreads);
          uint32_t r[32];
          tmem_ld_32x32(t_row + j * 32, r);
          tmem_ld_wait();
          uint8_t* row_ptr = buf + row_in_tile * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint4 v = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
            *reinterpret_cast<uint4*>(row_ptr + ((c ^ (row_in_tile & 7)) << 4)) = v;
          }
          fence_proxy_async_smem();
          named_bar_sync(1, kEpiThreads);
          if (leader) {
            if (n0 + j * 32 < N) {
              if (OUT == kOutF32Accum) tma_reduce_add_2d(&tmC, buf, n0 + j * 32, m0);
              else tma_store_2d(&tmC, buf, n0 + j * 32, m0);
            }
            tma_store_commit();
          }
          ++store_count;
        }
      }
      tc_fence_before();
      mbar_arrive(&sh->tmem_empty[acc]);
    }
    if (*(volatile int*)&sh->epi_abort && leader) {
      sh->abort_flag = 1;
      atomicCAS(err, 0, kErrEpilogue);
    }
    if (leader) {
      tma_store_wait_all<0>();
      if ((FUSE == kFuseRS || FUSE == kFuseAR) && pending_flag != nullptr) {
        fence_proxy_async_all();
        st_release_sys(pending_flag, fuse.epoch);
      }
    }
  }

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
    tmem_dealloc<Cfg::kTmemCols>(tmem_base);
  }
  if (FUSE == kFuseRS || FUSE == kFuseAR) {
    // the main loop is done: this CTA now helps summing the staged tiles its rank owns (the
    // dedicated CTAs [0, n_comm) have been doing so since launch)
    __syncthreads();
    rs_reduce_role<BN>(fuse, N, tiles_n, err, smem, (int)gridDim.x, false, FUSE == kFuseAR);
  }
  if (FUSE == kFuseAG && threadIdx.x == 0) {
    // last GEMM CTA of this rank: tell every peer that its pushes of this epoch were consumed
    __threadfence();
    const unsigned int old = atomicAdd(fuse.counter, 1u);
    if (old + 1 - fuse.counter_base == (unsigned int)cta_stride) {
      for (int p = 0; p < fuse.tp; ++p)
        if (p != fuse.rank) st_release_sys(fuse.done_ptrs[p] + fuse.rank, fuse.epoch);
    }
  }
}

// ---------------------------------- host side ------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows of `row_stride_bytes`.
static int make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* ptr, uint64_t inner, uint64_t outer,
                        uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                      uint32_t box_inner, uint32_t box_outer) {
  return make_tmap_2d(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ptr, inner, outer, row_stride_bytes, box_inner, box_outer);
}

int make_tmap_f32_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                     uint32_t box_inner, uint32_t box_outer) {
  return make_tmap_2d(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, ptr, inner, outer, row_stride_bytes, box_inner, box_outer);
}

static int make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* ptr, uint64_t inner, uint64_t outer,
                        uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -10;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (row_stride_bytes & 15)) return -11;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

template <int BN, bool A_MN, bool B_MN, int OUT, bool HAS_BIAS, int FUSE = kFuseNone>
static int launch_gemm(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC, const FuseArgs& fuse,
                       const __nv_bfloat16* bias, int M, int N, int K, int ldc, int* err, int max_ctas,
                       cudaStream_t stream, const CUtensorMap* tA2 = nullptr) {
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OUT, HAS_BIAS, FUSE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
  int grid = (FUSE != kFuseNone || tiles >= max_ctas) ? max_ctas : tiles;   // fused launches keep a fixed grid
  kern<<<grid, kGemmThreads, GemmCfg<BN>::kSmemBytes, stream>>>(tA, tB, tC, tA2 ? *tA2 : tA, fuse, bias, M, N, K, ldc,
                                                                err);
  return launch_status();
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = kNumSMs;
  }
  return n;
}

}  // namespace ell

using namespace ell;

// Self-test of the bounded peer-flag wait used by the fused kernels: one thread waits for *flag >= want exactly as a
// GEMM CTA waits for a peer's tile; if nothing raises the flag the wait gives up after its limit, the kernel records
// kErrFlagWait in *err and returns normally (no trap, the context stays usable).  Also covers the mbarrier wait
// (a barrier nobody arrives on) with the same limit.  *waited_ns receives the time spent in the two waits.
__global__ void bounded_wait_selftest_kernel(const uint32_t* flag, uint32_t want, int* err,
                                             unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x != 0) return;
  abort_flag = 0;
  mbar_init(&bar, 1);
  fence_barrier_init();
  const unsigned long long t0 = globaltimer_ns();
  const bool got_flag = wait_flag_ge(flag, want, &abort_flag);
  if (!got_flag) atomicCAS(err, 0, kErrFlagWait);
  const bool got_bar = got_flag ? true : mbar_wait(&bar, 0, &abort_flag);   // phase 0 never completes
  if (!got_bar) atomicCAS(err, 0, kErrProducer);
  *waited_ns = globaltimer_ns() - t0;
}

ELL_API int ell_bounded_wait_selftest(const void* flag, unsigned int want, int* err, unsigned long long* waited_ns,
                                      cudaStream_t stream) {
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>((const uint32_t*)flag, want, err, waited_ns);
  return launch_status();
}

namespace ell {
int g_no_tail_split = 0;   // shared with gemm_pair.cu
int g_rs_lag_q = 0;
unsigned long long g_fuse_data_bytes = 0;
}
// Size in bytes of each gathered / staging buffer of the fused-TP workspace: the fused kernels check every tile offset
// they compute against it (0 switches the offset check off; flag indices are always checked).
ELL_API void ell_gemm_set_fused_buffer_bytes(unsigned long long bytes) { ell::g_fuse_data_bytes = bytes; }
// Tuning switch: 0 (default) cuts the tiles of an under-filled last wave in two, 1 keeps whole tiles.
ELL_API void ell_gemm_set_tail_split(int enabled) { g_no_tail_split = enabled ? 0 : 1; }

template <int BN, int FUSE>
static int enumerate_units(int M, int N, const FuseArgs& f, int ctas, bool allow_split, int* out, int max_units) {
  const int tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int n_split = split_tail_tiles(num_tiles, ctas, FUSE == kFuseNone && BN == 256 && allow_split);
  const int num_full = num_tiles - n_split, num_units = num_tiles + n_split;
  if (num_units > max_units) return -1;
  for (int u = 0; u < num_units; ++u) {
    const TileUnit t = decode_unit<BN, FUSE>(u, tiles_m, tiles_n, num_full, f);
    out[4 * u + 0] = t.mt;
    out[4 * u + 1] = t.nt;
    out[4 * u + 2] = t.n0;
    out[4 * u + 3] = t.bn;
  }
  return num_units;
}

// Host-only: the work units of a launch in the order the kernel walks them (unit u goes to GEMM CTA u % ctas as its
// (u / ctas)-th item), computed by the kernel's own tile-order code.  out[u] = {row tile, column tile, first column,
// width}.  fuse: 0 plain, 1 all-gather -> GEMM, 2 GEMM -> reduce-scatter.  Returns the unit count, -1 if out is too
// small, -3 for an unsupported bn / fuse.  Touches no GPU.
ELL_API int ell_gemm_enumerate_units(int M, int N, int bn, int fuse, int tp, int rank, int ctas, int allow_split,
                                     int* out, int max_units) {
  FuseArgs f{};
  f.tp = tp;
  f.rank = rank;
  if (bn == 256 && fuse == kFuseNone) return enumerate_units<256, kFuseNone>(M, N, f, ctas, allow_split != 0, out, max_units);
  if (bn == 128 && fuse == kFuseNone) return enumerate_units<128, kFuseNone>(M, N, f, ctas, allow_split != 0, out, max_units);
  if (bn == 256 && fuse == kFuseAG) return enumerate_units<256, kFuseAG>(M, N, f, ctas, false, out, max_units);
  if (bn == 128 && fuse == kFuseAG) return enumerate_units<128, kFuseAG>(M, N, f, ctas, false, out, max_units);
  if (bn == 256 && fuse == kFuseRS) return enumerate_units<256, kFuseRS>(M, N, f, ctas, false, out, max_units);
  if (bn == 128 && fuse == kFuseRS) return enumerate_units<128, kFuseRS>(M, N, f, ctas, false, out, max_units);
  return -3;
}

// C = op(A)·op(B)^T.  a_mn / b_mn select MN-major storage ([K,M] / [K,N] row-major).
// out_mode: 0 bf16 C (ldc in elements), 1 fp32 C += result, 2 fp32 C = result.
// `err` is a device int that receives a non-zero code if a bounded wait inside the kernel expired.
ELL_API int ell_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                          int ldb, int ldc, int a_mn, int b_mn, int out_mode, int bn_hint, int* err,
                          cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (bias && out_mode != kOutBf16) return -2;
  if (out_mode == kOutBf16CE) return -2;   // needs the statistics arguments: use ell_gemm_ce
  int BN = (bn_hint == 128 || bn_hint == 256) ? bn_hint : (N >= 256 ? 256 : 128);
  CUtensorMap tA, tB, tC;
  int rc;
  if (!a_mn) rc = make_tmap_bf16_2d(&tA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, kBK, kBM);
  else       rc = make_tmap_bf16_2d(&tA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, kBK);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_bf16_2d(&tB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kBK, BN);
  else       rc = make_tmap_bf16_2d(&tB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, kBK);
  if (rc) return rc;
  if (out_mode == kOutBf16) {
    rc = make_tmap_bf16_2d(&tC, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64, 128);
    if (rc) return rc;
  } else {
    rc = make_tmap_f32_2d(&tC, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 4, 32, 128);
    if (rc) return rc;
  }
  const int ctas = sm_count();
  FuseArgs Cf{};
  Cf.no_tail_split = g_no_tail_split;
  const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(bias);
  // second B map with a box of BN/2 rows: used by the half-width tiles of a split tail wave
  CUtensorMap tBh = tB;
  if (!b_mn && BN == 256) {
    rc = make_tmap_bf16_2d(&tBh, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kBK, BN / 2);
    if (rc) return rc;
  }
#define ELL_GEMM_CASE(BN_, AM_, BM_, OUT_, BIAS_)                                                             \
  if (BN == BN_ && (bool)a_mn == AM_ && (bool)b_mn == BM_ && out_mode == OUT_ && (bias != nullptr) == BIAS_) \
    return launch_gemm<BN_, AM_, BM_, OUT_, BIAS_>(tA, tB, tC, Cf, bp, M, N, K, ldc, err, ctas, stream, &tBh);
#define ELL_GEMM_BN(BN_)                           \
  ELL_GEMM_CASE(BN_, false, false, kOutBf16, false) \
  ELL_GEMM_CASE(BN_, false, false, kOutBf16, true)  \
  ELL_GEMM_CASE(BN_, false, true, kOutBf16, false)  \
  ELL_GEMM_CASE(BN_, true, true, kOutBf16, false)   \
  ELL_GEMM_CASE(BN_, true, true, kOutF32Accum, false) \
  ELL_GEMM_CASE(BN_, true, true, kOutF32, false)    \
  ELL_GEMM_CASE(BN_, false, false, kOutF32, false)  \
  ELL_GEMM_CASE(BN_, false, true, kOutF32, false)
  ELL_GEMM_BN(256)
  ELL_GEMM_BN(128)
  return -3;
}

// Column tiles the cross-entropy epilogue produces partials for (BN = 256).
ELL_API int ell_gemm_ce_tiles(int N) { return (N + 255) / 256; }

// logits[M, N] (bf16) = X[M, K] · W[N, K]^T and, fused into the epilogue, per-(row, column tile) partial
// statistics part[tiles_n][3][M] = (max, sum exp(x - max), logit of the target if it falls in the tile else 0)
// over the first `valid_cols` columns; target holds global vocabulary ids, column 0 is id vocab_start.
ELL_API int ell_gemm_ce(const void* X, const void* W, void* logits, const long long* target, float* part, int M, int N,
                        int K, long long vocab_start, int valid_cols, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap tA, tB, tC;
  int rc = make_tmap_bf16_2d(&tA, X, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kBK, kBM);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tB, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, kBK, 256);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tC, logits, (uint64_t)N, (uint64_t)M, (uint64_t)N * 2, 64, 128);
  if (rc) return rc;
  FuseArgs f{};
  f.ce_target = target;
  f.ce_part = part;
  f.ce_vocab_start = vocab_start;
  f.ce_valid = valid_cols < N ? valid_cols : N;
  return launch_gemm<256, false, false, kOutBf16CE, false>(tA, tB, tC, f, nullptr, M, N, K, N, err, sm_count(), stream);
}

static void fill_fuse(FuseArgs& f, int rank, int tp, int n_comm, int rows_per_rank, int flags_per_src,
                      unsigned int epoch, void* const* data_ptrs, void* const* flag_ptrs, void* const* red_ptrs,
                      void* const* done_ptrs, void* counter, unsigned int counter_base) {
  f.rank = rank; f.tp = tp; f.n_comm = n_comm; f.rows_per_rank = rows_per_rank; f.flags_per_src = flags_per_src;
  f.epoch = epoch;
  for (int i = 0; i < tp; ++i) {
    f.data_ptrs[i] = (__nv_bfloat16*)data_ptrs[i];
    f.flag_ptrs[i] = (uint32_t*)flag_ptrs[i];
    f.red_ptrs[i] = red_ptrs ? (uint32_t*)red_ptrs[i] : nullptr;
    f.done_ptrs[i] = (uint32_t*)done_ptrs[i];
  }
  f.counter = (unsigned int*)counter;
  f.counter_base = counter_base;
  f.queue = f.counter + 1;
  f.data_bytes = g_fuse_data_bytes;
}

// Total CTAs of a fused single-CTA launch (communication CTAs included): the host advances its copy of the CTA
// counter by this (reduce forms) or by this minus n_comm (gather forms) per launch.
ELL_API int ell_gemm_fused_grid() { return sm_count(); }

// All-gather -> GEMM.  out[tp*rows_per_rank, N] = gather(x_local)[.., K] · W[N, K]^T (+ bias), or with
// b_mn = 1, gather(x_local) · W[K, N] (W read in place as an MN-major operand).
// gathered_ptrs[r] is rank r's gathered buffer [tp*rows_per_rank, K] (peer pointers; entry `rank` is local);
// flag_ptrs[r] / done_ptrs[r] are rank r's flag ([tp][flags_per_src]) and done ([tp]) words.  `counter_base` is the
// running value of the CTA counter: every launch advances it by (ell_gemm_fused_grid() - n_comm).
ELL_API int ell_gemm_ag(const void* x_local, const void* W, void* out, const void* bias, int rows_per_rank, int N,
                        int K, int b_mn, int rank, int tp, unsigned int epoch, int n_comm, void* const* gathered_ptrs,
                        void* const* flag_ptrs, void* const* done_ptrs, void* counter, unsigned int counter_base,
                        int flags_per_src, int* err, cudaStream_t stream) {
  if (tp < 1 || tp > kMaxTp || rows_per_rank % kBM || rows_per_rank / kBM > flags_per_src) return -2;
  if (b_mn && bias) return -2;
  const int M = rows_per_rank * tp;
  const int BN = N >= 256 ? 256 : 128;
  CUtensorMap tA, tB, tC;
  int rc = make_tmap_bf16_2d(&tA, gathered_ptrs[rank], (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kBK, kBM);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_bf16_2d(&tB, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, kBK, BN);
  else       rc = make_tmap_bf16_2d(&tB, W, (uint64_t)N, (uint64_t)K, (uint64_t)N * 2, 64, kBK);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tC, out, (uint64_t)N, (uint64_t)M, (uint64_t)N * 2, 64, 128);
  if (rc) return rc;
  CUtensorMap tA2;
  rc = make_tmap_bf16_2d(&tA2, x_local, (uint64_t)K, (uint64_t)rows_per_rank, (uint64_t)K * 2, kBK, kBM);
  if (rc) return rc;
  FuseArgs f{};
  fill_fuse(f, rank, tp, n_comm, rows_per_rank, flags_per_src, epoch, gathered_ptrs, flag_ptrs, nullptr, done_ptrs,
            counter, counter_base);
  f.x_local = (const __nv_bfloat16*)x_local;
  const int ctas = sm_count();
  if (n_comm < 1 || n_comm >= ctas) return -2;
  const __nv_bfloat16* bp = (const __nv_bfloat16*)bias;
  if (b_mn) {   // W is [K, N] row-major: the dgrad of a row-parallel linear (gathered dy · W)
    if (BN == 256) return launch_gemm<256, false, true, kOutBf16, false, kFuseAG>(tA, tB, tC, f, bp, M, N, K, N, err, ctas, stream, &tA2);
    return launch_gemm<128, false, true, kOutBf16, false, kFuseAG>(tA, tB, tC, f, bp, M, N, K, N, err, ctas, stream, &tA2);
  }
  if (BN == 256) {
    if (bias) return launch_gemm<256, false, false, kOutBf16, true, kFuseAG>(tA, tB, tC, f, bp, M, N, K, N, err, ctas, stream, &tA2);
    return launch_gemm<256, false, false, kOutBf16, false, kFuseAG>(tA, tB, tC, f, bp, M, N, K, N, err, ctas, stream, &tA2);
  }
  if (bias) return launch_gemm<128, false, false, kOutBf16, true, kFuseAG>(tA, tB, tC, f, bp, M, N, K, N, err, ctas, stream, &tA2);
  return launch_gemm<128, false, false, kOutBf16, false, kFuseAG>(tA, tB, tC, f, bp, M, N, K, N, err, ctas, stream, &tA2);
}

// GEMM -> reduce-scatter.  y_local[rows_per_rank, N] = sum over ranks of (x[M, K] · op(W))[own rows]; with
// all_reduce = 1, GEMM -> all-reduce: y is the full [M, N] sum on every rank and red_ptrs[r] rank r's "tile reduced"
// flags ([tp][flags_per_src]).
// b_mn = 0: W is [N, K] (forward of a row-parallel linear); b_mn = 1: W is [K, N] (its use as dgrad of a
// column-parallel linear).  stage_ptrs[r] is rank r's staging buffer [M, N].  `queue_base` is the running value
// of the tile queue: every launch advances it by ell_gemm_rs_queue_advance(...); `counter_base` that of the CTA
// counter, advanced by ell_gemm_fused_grid() per launch.
ELL_API int ell_gemm_rs(const void* x, const void* W, void* y_local, int rows_per_rank, int N, int K, int b_mn,
                        int rank, int tp, unsigned int epoch, int n_comm, void* const* stage_ptrs,
                        void* const* flag_ptrs, void* const* red_ptrs, void* const* done_ptrs, void* counter,
                        unsigned int counter_base, int flags_per_src, unsigned int queue_base, int all_reduce, int* err,
                        cudaStream_t stream) {
  if (tp < 1 || tp > kMaxTp || rows_per_rank % kBM || N % 8) return -2;
  if (all_reduce && !red_ptrs) return -2;
  const int M = rows_per_rank * tp;
  const int BN = N >= 256 ? 256 : 128;
  const int tiles_n = (N + BN - 1) / BN;
  if ((rows_per_rank / kBM) * tiles_n > flags_per_src) return -2;
  CUtensorMap tA, tB, tC;
  int rc = make_tmap_bf16_2d(&tA, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kBK, kBM);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_bf16_2d(&tB, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, kBK, BN);
  else       rc = make_tmap_bf16_2d(&tB, W, (uint64_t)N, (uint64_t)K, (uint64_t)N * 2, 64, kBK);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tC, stage_ptrs[rank], (uint64_t)N, (uint64_t)M, (uint64_t)N * 2, 64, 128);
  if (rc) return rc;
  FuseArgs f{};
  fill_fuse(f, rank, tp, n_comm, rows_per_rank, flags_per_src, epoch, stage_ptrs, flag_ptrs, red_ptrs, done_ptrs,
            counter, counter_base);
  f.y_local = (__nv_bfloat16*)y_local;
  f.queue_base = queue_base;
  const int ctas = sm_count();
  if (n_comm < 0 || n_comm >= ctas) return -2;
#define ELL_RS_CASE(BN_, BM_, FUSE_)                                                                        \
  if (BN == BN_ && (bool)b_mn == BM_ && (all_reduce ? kFuseAR : kFuseRS) == FUSE_)                          \
    return launch_gemm<BN_, false, BM_, kOutBf16, false, FUSE_>(tA, tB, tC, f, nullptr, M, N, K, N, err, ctas, stream);
  ELL_RS_CASE(256, false, kFuseRS)
  ELL_RS_CASE(256, true, kFuseRS)
  ELL_RS_CASE(128, false, kFuseRS)
  ELL_RS_CASE(128, true, kFuseRS)
  ELL_RS_CASE(256, false, kFuseAR)
  ELL_RS_CASE(256, true, kFuseAR)
  ELL_RS_CASE(128, false, kFuseAR)
  ELL_RS_CASE(128, true, kFuseAR)
#undef ELL_RS_CASE
  return -3;
}

// Queue positions one reduce launch consumes: the tiles it hands out (the owned ones; with all_reduce every tile of
// the output) plus one overshoot per CTA.  grid: ell_gemm_fused_grid() or ell_gemm_pair_fused_grid().
ELL_API int ell_gemm_rs_queue_advance(int rows_per_rank, int N, int tp, int all_reduce, int grid) {
  const int BN = N >= 256 ? 256 : 128;
  const int owned = (rows_per_rank / kBM) * ((N + BN - 1) / BN);
  return owned * (all_reduce ? tp : 1) + grid;
}
