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
#include "common.cuh"
#include "sm100.cuh"

namespace ell {
using namespace sm100;

constexpr int kBM = 128;
constexpr int kBK = 64;                    // 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kABytes = kBM * kBK * 2;     // 16 KiB
constexpr int kEpiBufBytes = 128 * 64 * 2; // one 128x64 bf16 store box

// kOutBf16CE: bf16 C plus, per row and column tile, the cross-entropy statistics (max, sum-exp, target logit)
// of the rounded logits, computed in the epilogue while the tile is in registers.
enum GemmOut { kOutBf16 = 0, kOutF32Accum = 1, kOutF32 = 2, kOutBf16CE = 3 };
enum GemmErr { kErrProducer = 1, kErrMma = 2, kErrEpilogue = 3, kErrComm = 4, kErrFlagWait = 5 };

// ---- fusion with the tensor-parallel collective (sequence parallelism) ------------------------------
//  kFuseAG  all-gather -> GEMM: the A operand is the concatenation over ranks of row shards.  CTAs
//           [0, n_comm) copy this rank's shard into every rank's gathered buffer through peer pointers
//           (plain 16-byte loads/stores over NVLink), one 128-row tile at a time, and publish a flag per
//           tile; the GEMM CTAs start on the local shard and take remote shards in ring order, waiting
//           on a tile's flag only before its first TMA load (always a load of local memory into one CTA).
//  kFuseRS  GEMM -> reduce-scatter: every rank computes the full partial product; finished bf16 tiles
//           go to a local staging buffer (TMA store) and a flag is raised on the tile's owner rank; CTAs
//           [0, n_comm) of the owner sum the tp staged copies (peer loads, fp32 add, fixed order so the
//           result is deterministic) into the local output shard while the main loop is still running,
//           and every GEMM CTA joins that reduction as soon as its own tiles are done.
// Flags are epoch counters that only grow; a per-peer `done` word tells a producer that the consumer
// has finished the previous epoch before a buffer is overwritten.  Every wait is bounded.
enum GemmFuse { kFuseNone = 0, kFuseAG = 1, kFuseRS = 2 };
constexpr int kMaxTp = 8;
constexpr int kGroupM = 16;   // tiles are walked in groups of 16 M-tiles x all N-tiles for L2 reuse

struct FuseArgs {
  int rank, tp, n_comm, rows_per_rank, flags_per_src;
  uint32_t epoch;
  const __nv_bfloat16* x_local;          // AG: this rank's shard [rows_per_rank, K]
  __nv_bfloat16* data_ptrs[kMaxTp];      // AG: gathered buffers [M, K]; RS: staging buffers [M, N]
  uint32_t* flag_ptrs[kMaxTp];           // [tp][flags_per_src] on every rank
  uint32_t* done_ptrs[kMaxTp];           // [tp] on every rank
  unsigned int* counter;                 // local, monotonic: finished CTAs
  unsigned int* queue;                   // RS: local, monotonic: next owned tile to reduce
  unsigned int queue_base;               // RS: value of *queue when this launch starts (tracked by the host)
  __nv_bfloat16* y_local;                // RS: output shard [rows_per_rank, N]
  // kOutBf16CE: targets [M] (global vocab ids), partials [tiles_n][3][M], first vocab id of column 0,
  // number of leading columns that are real vocabulary (the padded tail is excluded)
  const long long* ce_target;
  float* ce_part;
  long long ce_vocab_start;
  int ce_valid;
  int no_tail_split;                     // plain launches: 1 disables the half-width tail tiles
  int prefetch_kb;                       // L2 prefetch distance of the producer in k-blocks (0 = off)
  int rs_ring;                           // RS: 1 = ring tile order (own tiles last), 0 = owners interleaved
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded spin until *flag >= want.  False on timeout / abort.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want, volatile int* abort_flag) {
  if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while ((int32_t)(ld_acquire_sys(flag) - want) < 0) {
    if ((++spins & 63u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitTimeoutNs) return false;
    }
  }
  return true;
}

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
  } else if (FUSE == kFuseRS) {
    if (f.rs_ring) {
      // ring order: the tiles owned by rank+1 first, ..., this rank's own tiles last.  Partials for remote owners
      // cross NVLink early, and the tiles a rank reduces at the very end only wait for its own (local) partial.
      const int tpr = tiles_m / f.tp, per_phase = tpr * tiles_n;
      const int phase = idx / per_phase;
      int mi;
      swizzle_tile(idx % per_phase, tpr, tiles_n, mi, nt);
      mt = ((f.rank + 1 + phase) % f.tp) * tpr + mi;
    } else {
      int mp;
      swizzle_tile(idx, tiles_m, tiles_n, mp, nt);
      mt = (mp % f.tp) * (tiles_m / f.tp) + mp / f.tp;   // interleave owners so every owner is fed evenly
    }
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


// ---- communication roles (CTAs [0, n_comm) of a fused launch) ---------------------------------------
// Both roles move data with the bulk-copy engine (cp.async.bulk through a shared-memory ring), driven by
// one thread, so a CTA keeps ~190 KB in flight: NVLink latency is hidden without many threads or SMs.
constexpr int kCommStages = 6;
constexpr int kCommChunkBytes = 32768;

struct CommShared {
  uint64_t full[kCommStages];
  uint64_t empty[kCommStages];
  int meta[kCommStages];
  int abort_flag;
};

// All-gather side: copy the local shard, tile by tile, into the gathered buffer of every other rank.
// (The local GEMM reads its own shard in place; nothing is copied to self.)
__device__ void ag_comm_role(const FuseArgs& f, int K, int* err, uint8_t* smem) {
  CommShared* cs = reinterpret_cast<CommShared*>(smem + kCommStages * kCommChunkBytes);
  if (threadIdx.x != 0) return;
  for (int s = 0; s < kCommStages; ++s) mbar_init(&cs->full[s], 1);
  cs->abort_flag = 0;
  fence_barrier_init();
  volatile int* abort_flag = &cs->abort_flag;
  const int tiles = f.rows_per_rank / kBM;
  const size_t tile_bytes = (size_t)kBM * K * 2;
  const int chunks = (int)((tile_bytes + kCommChunkBytes - 1) / kCommChunkBytes);
  // destinations must have consumed the previous epoch before their buffers are overwritten
  for (int d = 0; d < f.tp; ++d)
    if (d != f.rank && !wait_flag_ge(f.done_ptrs[f.rank] + d, f.epoch - 1, abort_flag)) {
      atomicCAS(err, 0, kErrComm);
      return;
    }
  uint32_t issued = 0, landed = 0;   // chunk counters across items select ring stage and parity
  // Work item = (row tile, destination): with few row tiles per rank (large tp) every comm CTA still has work,
  // and each destination's flag is raised as soon as its copy of the tile has landed.
  const int n_dest = f.tp - 1;
  const int n_items = tiles * n_dest;
  for (int item = blockIdx.x; item < n_items; item += f.n_comm) {
    const int t = item / n_dest;
    const int dest = (f.rank - 1 - item % n_dest + f.tp) % f.tp;   // the rank that needs this shard soonest first
    const uint8_t* src = reinterpret_cast<const uint8_t*>(f.x_local) + (size_t)t * tile_bytes;
    uint8_t* dst = reinterpret_cast<uint8_t*>(f.data_ptrs[dest]) +
                   ((size_t)f.rank * f.rows_per_rank + (size_t)t * kBM) * K * 2;
    int next_load = 0;
    auto issue_load = [&](int c) {
      const uint32_t st = issued % kCommStages;
      const uint32_t bytes = (uint32_t)min((size_t)kCommChunkBytes, tile_bytes - (size_t)c * kCommChunkBytes);
      mbar_expect_tx(&cs->full[st], bytes);
      bulk_load(smem + st * kCommChunkBytes, src + (size_t)c * kCommChunkBytes, bytes, &cs->full[st]);
      ++issued;
    };
    for (; next_load < chunks && next_load < kCommStages - 1; ++next_load) issue_load(next_load);
    for (int c = 0; c < chunks; ++c) {
      const uint32_t st = landed % kCommStages;
      if (!mbar_wait(&cs->full[st], (landed / kCommStages) & 1, abort_flag)) {
        atomicCAS(err, 0, kErrComm);
        return;
      }
      ++landed;
      const uint32_t bytes = (uint32_t)min((size_t)kCommChunkBytes, tile_bytes - (size_t)c * kCommChunkBytes);
      bulk_store(dst + (size_t)c * kCommChunkBytes, smem + st * kCommChunkBytes, bytes);
      tma_store_commit();
      if (next_load < chunks) {
        tma_store_wait_read<1>();   // the stage about to be refilled was last read by the previous group
        issue_load(next_load++);
      }
    }
    tma_store_wait_all<0>();        // the whole tile has been written on the destination
    fence_proxy_async_all();
    __threadfence_system();
    st_release_sys(f.flag_ptrs[dest] + (size_t)f.rank * f.flags_per_src + t, f.epoch);
  }
}

// Staged tile layout of GEMM->reduce-scatter: every 128x64 bf16 sub-tile is one contiguous 16 KiB block
// (rows of 128 B, 16-byte chunks XOR-swizzled by row & 7, exactly as the epilogue wrote them to smem).
template <int BN>
__device__ __forceinline__ size_t stage_block(int mt, int nt, int j, int tiles_n) {
  return ((size_t)(mt * tiles_n + nt) * (BN / 64) + j) * kEpiBufBytes;
}

// Reduce-scatter side: sum the tp staged copies of every tile this rank owns into y_local.
// Owned tiles are handed out through a global queue in the order producers emit them, so the dedicated
// CTAs keep pace with the main loop and the GEMM CTAs only pick up what is left when they finish.
template <int BN>
__device__ void rs_reduce_role(const FuseArgs& f, int N, int tiles_n, int* err, uint8_t* smem, int nparts) {
  CommShared* cs = reinterpret_cast<CommShared*>(smem + kCommStages * kCommChunkBytes);
  constexpr int kConsumers = kGemmThreads - 32;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kCommStages; ++s) {
      mbar_init(&cs->full[s], 1);
      mbar_init(&cs->empty[s], kConsumers);
    }
    cs->abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  volatile int* abort_flag = &cs->abort_flag;
  const int tpr = f.rows_per_rank / kBM;
  const int owned = tpr * tiles_n;
  const int gm = f.rs_ring ? kGroupM : max(1, kGroupM / f.tp);   // the order in which producers emit owned tiles
  const int R = 256 / f.tp;                   // rows per ring stage: tp sources x R rows x 128 B = 32 KiB
  const int parts = kBM / R;
  const uint32_t src_bytes = (uint32_t)R * 128;
  const unsigned int queue_base = f.queue_base;
  if (threadIdx.x == 0) {
    uint32_t item = 0;
    bool ok = true;
    while (ok) {
      const int j = (int)(atomicAdd(f.queue, 1u) - queue_base);
      if (j >= owned) break;
      const int width = gm * tiles_n, g = j / width, rem = j % width;
      const int first = g * gm, gsz = min(tpr - first, gm);
      const int mi = first + rem % gsz, nt = rem / gsz;
      for (int s = 0; s < f.tp && ok; ++s) {
        const uint32_t* fl = f.flag_ptrs[f.rank] + (size_t)s * f.flags_per_src + mi * tiles_n + nt;
        ok = wait_flag_ge(fl, f.epoch, abort_flag);
      }
      if (!ok) break;
      fence_proxy_async_all();
      const int mt = f.rank * tpr + mi;
      for (int sub = 0; sub < BN / 64 && ok; ++sub) {
        const size_t blk = stage_block<BN>(mt, nt, sub, tiles_n);
        for (int p = 0; p < parts; ++p, ++item) {
          const uint32_t st = item % kCommStages;
          if (!mbar_wait(&cs->empty[st], ((item / kCommStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
          cs->meta[st] = ((mi * tiles_n + nt) * (BN / 64) + sub) * parts + p;
          mbar_expect_tx(&cs->full[st], src_bytes * f.tp);
          for (int s = 0; s < f.tp; ++s)
            bulk_load(smem + st * kCommChunkBytes + s * src_bytes,
                      reinterpret_cast<const uint8_t*>(f.data_ptrs[s]) + blk + (size_t)p * src_bytes, src_bytes,
                      &cs->full[st]);
        }
      }
    }
    if (ok) {
      // end marker for the consumers
      const uint32_t st = item % kCommStages;
      if (mbar_wait(&cs->empty[st], ((item / kCommStages) & 1) ^ 1, abort_flag)) {
        cs->meta[st] = -1;
        mbar_arrive(&cs->full[st]);
      } else {
        ok = false;
      }
    }
    if (!ok) {
      cs->abort_flag = 1;
      atomicCAS(err, 0, kErrComm);
    }
  } else if (threadIdx.x >= 32) {
    const int ct = threadIdx.x - 32;
    for (uint32_t item = 0;; ++item) {
      const uint32_t st = item % kCommStages;
      if (!mbar_wait(&cs->full[st], (item / kCommStages) & 1, abort_flag)) break;
      int code = cs->meta[st];
      if (code < 0) break;
      const int p = code % parts; code /= parts;
      const int sub = code % (BN / 64); code /= (BN / 64);
      const int nt = code % tiles_n, mi = code / tiles_n;
      const uint8_t* base = smem + st * kCommChunkBytes;
      for (int q = ct; q < R * 8; q += kConsumers) {
        const int rl = q >> 3, cphys = q & 7;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int s = 0; s < f.tp; ++s) {
          float t[8];
          unpack8(*reinterpret_cast<const bf16x8*>(base + s * src_bytes + q * 16), t);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += t[e];
        }
        const int row = p * R + rl;
        const int col = nt * BN + sub * 64 + ((cphys ^ (row & 7)) << 3);
        if (col < N) *reinterpret_cast<bf16x8*>(f.y_local + ((size_t)mi * kBM + row) * N + col) = pack8(acc);
      }
      mbar_arrive(&cs->empty[st]);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int old = atomicAdd(f.counter, 1u);
    if ((old + 1) % (unsigned int)nparts == 0) {
      for (int p = 0; p < f.tp; ++p)
        if (p != f.rank) st_release_sys(f.done_ptrs[p] + f.rank, f.epoch);
    }
  }
}

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
    if (FUSE == kFuseAG) ag_comm_role(fuse, K, err, smem);
    else rs_reduce_role<BN>(fuse, N, tiles_n, err, smem, (int)gridDim.x);
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
          // optional L2 prefetch of the k-block `prefetch_kb` ahead (off by default: on B200 it slowed every shape,
          // the CTAs that share a tile each re-request it)
          if (FUSE != kFuseAG && fuse.prefetch_kb > 0 && kb + fuse.prefetch_kb < num_kb) {
            const int kp = (kb + fuse.prefetch_kb) * kBK;
            if (!A_MN) {
              tma_prefetch_l2_2d(a_map, kp, a_row);
            } else {
#pragma unroll
              for (int i = 0; i < kBM / 64; ++i) tma_prefetch_l2_2d(&tmA, m0 + i * 64, kp);
            }
            if (!B_MN) {
              tma_prefetch_l2_2d(b_map, kp, n0);
            } else {
#pragma unroll
              for (int i = 0; i < BN / 64; ++i)
                if (i * 64 < u.bn) tma_prefetch_l2_2d(&tmB, n0 + i * 64, kp);
            }
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
    if (FUSE == kFuseRS && leader) {
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
            if (FUSE == kFuseRS) {
              bulk_store(reinterpret_cast<uint8_t*>(fuse.data_ptrs[fuse.rank]) + stage_block<BN>(mt, nt, j, tiles_n),
                         buf, kEpiBufBytes);
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
        if (FUSE == kFuseRS && leader) {
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
      if (FUSE == kFuseRS && pending_flag != nullptr) {
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
  if (FUSE == kFuseRS) {
    // the main loop is done: this CTA now helps summing the staged tiles its rank owns (the
    // dedicated CTAs [0, n_comm) have been doing so since launch)
    __syncthreads();
    rs_reduce_role<BN>(fuse, N, tiles_n, err, smem, (int)gridDim.x);
  }
  if (FUSE == kFuseAG && threadIdx.x == 0) {
    // last GEMM CTA of this rank: tell every peer that its pushes of this epoch were consumed
    __threadfence();
    const unsigned int old = atomicAdd(fuse.counter, 1u);
    if ((old + 1) % (unsigned int)cta_stride == 0) {
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
}
static int g_rs_ring = 0;   // measured on 2 x B200: the ring order is not faster (o_proj 0.103 vs 0.101 ms, down 0.183 vs 0.177)
// Tuning switch: tile order of the GEMM -> reduce-scatter kernel (1 ring order, 0 owners interleaved).
ELL_API void ell_gemm_set_rs_order(int ring) { g_rs_ring = ring ? 1 : 0; }
static int g_prefetch_kb = 0;   // measured on B200: distances 4-16 cost 15-40 % (every CTA re-requests shared tiles)
// Tuning switch: L2 prefetch distance of the GEMM producer in 64-element k-blocks (0 disables it).
ELL_API void ell_gemm_set_prefetch(int k_blocks) { g_prefetch_kb = k_blocks < 0 ? 0 : k_blocks; }

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
ELL_API int ell_gemm_enumerate_units(int M, int N, int bn, int fuse, int tp, int rank, int rs_ring, int ctas,
                                     int allow_split, int* out, int max_units) {
  FuseArgs f{};
  f.tp = tp;
  f.rank = rank;
  f.rs_ring = rs_ring;
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
  Cf.prefetch_kb = g_prefetch_kb;
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
  f.prefetch_kb = g_prefetch_kb;
  return launch_gemm<256, false, false, kOutBf16CE, false>(tA, tB, tC, f, nullptr, M, N, K, N, err, sm_count(), stream);
}

static void fill_fuse(FuseArgs& f, int rank, int tp, int n_comm, int rows_per_rank, int flags_per_src,
                      unsigned int epoch, void* const* data_ptrs, void* const* flag_ptrs, void* const* done_ptrs,
                      void* counter) {
  f.rank = rank; f.tp = tp; f.n_comm = n_comm; f.rows_per_rank = rows_per_rank; f.flags_per_src = flags_per_src;
  f.epoch = epoch;
  for (int i = 0; i < tp; ++i) {
    f.data_ptrs[i] = (__nv_bfloat16*)data_ptrs[i];
    f.flag_ptrs[i] = (uint32_t*)flag_ptrs[i];
    f.done_ptrs[i] = (uint32_t*)done_ptrs[i];
  }
  f.counter = (unsigned int*)counter;
  f.queue = f.counter + 1;
  f.prefetch_kb = g_prefetch_kb;
  f.rs_ring = g_rs_ring;
}

// All-gather -> GEMM.  out[tp*rows_per_rank, N] = gather(x_local)[.., K] · W[N, K]^T (+ bias), or with
// b_mn = 1, gather(x_local) · W[K, N] (W read in place as an MN-major operand).
// gathered_ptrs[r] is rank r's gathered buffer [tp*rows_per_rank, K] (peer pointers; entry `rank` is local);
// flag_ptrs[r] / done_ptrs[r] are rank r's flag ([tp][flags_per_src]) and done ([tp]) words.
ELL_API int ell_gemm_ag(const void* x_local, const void* W, void* out, const void* bias, int rows_per_rank, int N,
                        int K, int b_mn, int rank, int tp, unsigned int epoch, int n_comm, void* const* gathered_ptrs,
                        void* const* flag_ptrs, void* const* done_ptrs, void* counter, int flags_per_src, int* err,
                        cudaStream_t stream) {
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
  fill_fuse(f, rank, tp, n_comm, rows_per_rank, flags_per_src, epoch, gathered_ptrs, flag_ptrs, done_ptrs, counter);
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

// GEMM -> reduce-scatter.  y_local[rows_per_rank, N] = sum over ranks of (x[M, K] · op(W))[own rows].
// b_mn = 0: W is [N, K] (forward of a row-parallel linear); b_mn = 1: W is [K, N] (its use as dgrad of a
// column-parallel linear).  stage_ptrs[r] is rank r's staging buffer [M, N].  `queue_base` is the running value
// of the tile queue: every launch advances it by (owned tiles + number of CTAs); ell_gemm_rs_queue_advance
// returns that amount.
ELL_API int ell_gemm_rs(const void* x, const void* W, void* y_local, int rows_per_rank, int N, int K, int b_mn,
                        int rank, int tp, unsigned int epoch, int n_comm, void* const* stage_ptrs,
                        void* const* flag_ptrs, void* const* done_ptrs, void* counter, int flags_per_src,
                        unsigned int queue_base, int* err, cudaStream_t stream) {
  if (tp < 1 || tp > kMaxTp || rows_per_rank % kBM || N % 8) return -2;
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
  fill_fuse(f, rank, tp, n_comm, rows_per_rank, flags_per_src, epoch, stage_ptrs, flag_ptrs, done_ptrs, counter);
  f.y_local = (__nv_bfloat16*)y_local;
  f.queue_base = queue_base;
  const int ctas = sm_count();
  if (n_comm < 0 || n_comm >= ctas) return -2;
  if (BN == 256) {
    if (b_mn) return launch_gemm<256, false, true, kOutBf16, false, kFuseRS>(tA, tB, tC, f, nullptr, M, N, K, N, err, ctas, stream);
    return launch_gemm<256, false, false, kOutBf16, false, kFuseRS>(tA, tB, tC, f, nullptr, M, N, K, N, err, ctas, stream);
  }
  if (b_mn) return launch_gemm<128, false, true, kOutBf16, false, kFuseRS>(tA, tB, tC, f, nullptr, M, N, K, N, err, ctas, stream);
  return launch_gemm<128, false, false, kOutBf16, false, kFuseRS>(tA, tB, tC, f, nullptr, M, N, K, N, err, ctas, stream);
}

ELL_API int ell_gemm_rs_queue_advance(int rows_per_rank, int N) {
  const int BN = N >= 256 ? 256 : 128;
  return (rows_per_rank / kBM) * ((N + BN - 1) / BN) + sm_count();
}
