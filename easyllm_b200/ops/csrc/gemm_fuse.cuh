// Fusion of the tcgen05 GEMMs with the tensor-parallel collectives: arguments, flag protocol and the
// communication roles shared by the single-CTA kernel (gemm.cu) and the CTA-pair kernel (gemm_pair.cu).
//
//  kFuseAG   all-gather -> GEMM: the A operand is the concatenation over ranks of row shards.  CTAs
//            [0, n_comm) copy this rank's shard into every rank's gathered buffer through peer pointers
//            (bulk copies through a shared-memory ring over NVLink), one 128-row tile at a time, and publish
//            a flag per tile; the GEMM CTAs start on the local shard and take remote shards in ring order,
//            waiting on a tile's flag only before its first TMA load (always a load of local memory).
//  kFuseAGK  the same gather, but the gathered operand is B and the gathered rows are the REDUCTION dimension
//            (the weight-gradient GEMM dW = dy^T · gather(x)): every output tile walks the k-blocks starting
//            at the local shard and waits for a remote row tile before its first k-block that reads it.
//  kFuseRS   GEMM -> reduce-scatter: every rank computes the full partial product; finished bf16 tiles go to a
//            local staging buffer and a flag is raised on the tile's owner rank; CTAs [0, n_comm) of the owner
//            sum the tp staged copies (peer bulk loads, fp32 add in a fixed order, so the result is
//            deterministic) into the local output shard while the main loop is still running, and every GEMM
//            CTA joins that reduction as soon as its own tiles are done.
//  kFuseAR   GEMM -> all-reduce (the tensor-parallel path without sequence parallelism): the reduce-scatter
//            above, after which each owner leaves the reduced tile in its staging buffer and raises a second
//            flag on every peer; all ranks then pull the tiles they do not own (peer bulk loads) into their
//            full-size output.  Two-shot: each byte crosses NVLink once per phase.
// Flags are epoch counters that only grow; a per-peer `done` word tells a producer that the consumer has
// finished the previous epoch before a buffer is overwritten.  Every wait is bounded and reports through the
// error word.  Tensor maps only ever cover this GPU's memory and no load names more than one destination CTA.
//
// Replaces the separate collectives of llm/models/mg_models/base_modules/layers/column_parallel_linear.py:29-38,
// 53-61,87-95, row_parallel_linear.py:116-119 and llm/utils/env/dist_env/dist_mappings.py:48-58,125-162.
#pragma once
#include "common.cuh"
#include "sm100.cuh"

namespace ell {
using namespace sm100;

constexpr int kBM = 128;
constexpr int kBK = 64;                    // 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kEpiBufBytes = 128 * 64 * 2; // one 128x64 bf16 store box

// kOutBf16CE: bf16 C plus, per row and column slot, the cross-entropy statistics (max, sum-exp, target logit)
// of the rounded logits, computed in the epilogue while the tile is in registers.
enum GemmOut { kOutBf16 = 0, kOutF32Accum = 1, kOutF32 = 2, kOutBf16CE = 3 };
enum GemmErr { kErrProducer = 1, kErrMma = 2, kErrEpilogue = 3, kErrComm = 4, kErrFlagWait = 5, kErrBounds = 6 };
enum GemmFuse { kFuseNone = 0, kFuseAG = 1, kFuseRS = 2, kFuseAR = 3, kFuseAGK = 4 };
constexpr int kMaxTp = 8;

struct FuseArgs {
  int rank, tp, n_comm, rows_per_rank, flags_per_src;
  uint32_t epoch;
  const __nv_bfloat16* x_local;          // AG / AGK: this rank's shard [rows_per_rank, K]
  __nv_bfloat16* data_ptrs[kMaxTp];      // AG / AGK: gathered buffers [M, K]; RS / AR: staging buffers [M, N]
  uint32_t* flag_ptrs[kMaxTp];           // [tp][flags_per_src] on every rank
  uint32_t* red_ptrs[kMaxTp];            // AR: [tp][flags_per_src] on every rank, "owner has reduced this tile"
  uint32_t* done_ptrs[kMaxTp];           // [tp] on every rank
  unsigned int* counter;                 // local, monotonic: finished CTAs
  unsigned int counter_base;             // value of *counter when this launch starts (tracked by the host)
  unsigned int* queue;                   // RS / AR: local, monotonic: next tile to reduce / fetch
  unsigned int queue_base;               // RS / AR: value of *queue when this launch starts (tracked by the host)
  __nv_bfloat16* y_local;                // RS: output shard [rows_per_rank, N]; AR: full output [M, N]
  // kOutBf16CE: targets [M] (global vocab ids), partials [slots][3][M], first vocab id of column 0,
  // number of leading columns that are real vocabulary (the padded tail is excluded)
  const long long* ce_target;
  float* ce_part;
  long long ce_vocab_start;
  int ce_valid;
  int no_tail_split;                     // 1 disables the half-width units of an under-filled last wave
  int shard_k;                           // row length of x_local when this struct describes a bare push (see below)
  int k_passes;                          // AGK: 2 walks every tile twice (local half of the k-range first), 1 once
  unsigned long long data_bytes;         // size of each data_ptrs[] buffer: every computed offset is checked against it
  int rs_lag_q;                          // CTA-pair reduce-scatter: own tiles trail the peers' by this many quarter waves (0: default)
};

// Tile-granular bounds check of the fused kernels (always on: a few compares per 128-row tile).  A tile whose flag
// index or buffer offset falls outside what the host allocated is reported (kErrBounds) and skipped, never accessed.
__device__ __forceinline__ bool fuse_in_bounds(const FuseArgs& f, long long flag_idx, unsigned long long end_offset,
                                               int* err) {
  if (flag_idx < 0 || flag_idx >= f.flags_per_src || (f.data_bytes != 0 && end_offset > f.data_bytes)) {
    atomicCAS(err, 0, kErrBounds);
    return false;
  }
  return true;
}

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
// (The local GEMM reads its own shard in place; nothing is copied to self.)  `K` is the row length of the shard;
// CTAs [first_cta, first_cta + n_ctas) of the grid share the work.
// A reduce-scatter launch can carry such a push for the NEXT kernel on the stream (the weight-gradient GEMM that
// follows a dgrad -> reduce-scatter needs the gathered x): its transfer then hides behind this kernel's main loop.
__device__ inline void ag_comm_role(const FuseArgs& f, int K, int* err, uint8_t* smem, int first_cta, int n_ctas) {
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
  for (int item = (int)blockIdx.x - first_cta; item < n_items; item += n_ctas) {
    const int t = item / n_dest;
    const int dest = (f.rank - 1 - item % n_dest + f.tp) % f.tp;   // the rank that needs this shard soonest first
    const uint8_t* src = reinterpret_cast<const uint8_t*>(f.x_local) + (size_t)t * tile_bytes;
    const size_t dst_off = ((size_t)f.rank * f.rows_per_rank + (size_t)t * kBM) * K * 2;
    if (!fuse_in_bounds(f, t, dst_off + tile_bytes, err)) return;
    uint8_t* dst = reinterpret_cast<uint8_t*>(f.data_ptrs[dest]) + dst_off;
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
// `mt` counts 128-row tiles, `nt` column tiles of BN columns.
template <int BN>
__host__ __device__ __forceinline__ size_t stage_block(int mt, int nt, int j, int tiles_n) {
  return ((size_t)(mt * tiles_n + nt) * (BN / 64) + j) * kEpiBufBytes;
}

// Queue position -> owned 128-row tile, in the order the producers of this kernel family emit them, so the
// dedicated reduce CTAs keep pace with the main loops instead of waiting for a late tile while early ones sit
// ready.  group_m: row tiles per raster group and owner (single-CTA: 16 / tp 128-row tiles; CTA pair: 8 / tp
// 256-row tiles, each of which yields two consecutive 128-row tiles).
__host__ __device__ __forceinline__ void owned_tile_of(int j, int tpr, int tiles_n, int tp, bool pair, int& mi, int& nt) {
  const int unit_rows = pair ? 2 : 1;
  const int jj = j / unit_rows, h = j % unit_rows;
  const int tpr_u = tpr / unit_rows;
  const int group = pair ? 8 : 16;
  const int gm = group / tp > 0 ? group / tp : 1;
  const int width = gm * tiles_n, g = jj / width, rem = jj % width;
  const int first = g * gm;
  const int gsz = (tpr_u - first) < gm ? (tpr_u - first) : gm;
  const int mu = first + rem % gsz;
  nt = rem / gsz;
  mi = mu * unit_rows + h;
}

// Reduce-scatter / all-reduce side.  Phase 1: sum the tp staged copies of every tile this rank owns into y.
// Phase 2 (all-reduce only): fetch the reduced tiles of the other owners.  Tiles are handed out through a global
// queue, so the dedicated CTAs keep pace with the main loop and the GEMM CTAs only pick up what is left when they
// finish.  One thread drives the bulk loads, 160 threads add and store.
template <int BN>
__device__ inline void rs_reduce_role(const FuseArgs& f, int N, int tiles_n, int* err, uint8_t* smem, int nparts,
                                      bool pair, bool all_reduce) {
  CommShared* cs = reinterpret_cast<CommShared*>(smem + kCommStages * kCommChunkBytes);
  constexpr int kConsumers = kGemmThreads - 32;
  constexpr int kSub = BN / 64;
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
  const int total = all_reduce ? owned * f.tp : owned;
  const int R = f.tp >= 2 ? 256 / f.tp : kBM; // rows per ring stage in phase 1: tp sources x R rows x 128 B <= 32 KiB
  const int parts = kBM / R;
  const uint32_t src_bytes = (uint32_t)R * 128;
  const unsigned int queue_base = f.queue_base;
  // meta code of a ring stage: phase 1: ((tile * kSub + sub) * parts + p) * 2; phase 2: ((o * owned + tile) * kSub + sub) * 2 + 1;
  // bit 30 marks the last stage of a tile (all-reduce: the consumers then publish the reduced tile)
  if (threadIdx.x == 0) {
    uint32_t item = 0;
    bool ok = true;
    while (ok) {
      const int j = (int)(atomicAdd(f.queue, 1u) - queue_base);
      if (j >= total) break;
      if (j < 0) {   // the host's copy of the queue ran ahead of the device's: refuse to index with it
        ok = false;
        break;
      }
      if (j < owned) {
        int mi, nt;
        owned_tile_of(j, tpr, tiles_n, f.tp, pair, mi, nt);
        if (mi < 0 || mi >= tpr || nt < 0 || nt >= tiles_n ||
            !fuse_in_bounds(f, (long long)mi * tiles_n + nt,
                            stage_block<BN>(f.rank * tpr + mi, nt, kSub - 1, tiles_n) + kEpiBufBytes, err)) {
          ok = false;
          break;
        }
        for (int s = 0; s < f.tp && ok; ++s) {
          const uint32_t* fl = f.flag_ptrs[f.rank] + (size_t)s * f.flags_per_src + mi * tiles_n + nt;
          ok = wait_flag_ge(fl, f.epoch, abort_flag);
        }
        if (!ok) break;
        fence_proxy_async_all();
        const int mt = f.rank * tpr + mi;
        for (int sub = 0; sub < kSub && ok; ++sub) {
          const size_t blk = stage_block<BN>(mt, nt, sub, tiles_n);
          for (int p = 0; p < parts; ++p, ++item) {
            const uint32_t st = item % kCommStages;
            if (!mbar_wait(&cs->empty[st], ((item / kCommStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
            const bool last = (sub == kSub - 1) && (p == parts - 1);
            cs->meta[st] = ((((mi * tiles_n + nt) * kSub + sub) * parts + p) << 1) | (last ? (1 << 30) : 0);
            mbar_expect_tx(&cs->full[st], src_bytes * f.tp);
            for (int s = 0; s < f.tp; ++s)
              bulk_load(smem + st * kCommChunkBytes + s * src_bytes,
                        reinterpret_cast<const uint8_t*>(f.data_ptrs[s]) + blk + (size_t)p * src_bytes, src_bytes,
                        &cs->full[st]);
          }
        }
      } else {
        // phase 2: a tile another rank owns, once that rank has published its sum
        const int j2 = j - owned;
        const int o = (f.rank + 1 + j2 / owned) % f.tp;
        int mi, nt;
        owned_tile_of(j2 % owned, tpr, tiles_n, f.tp, pair, mi, nt);
        if (mi < 0 || mi >= tpr || nt < 0 || nt >= tiles_n ||
            !fuse_in_bounds(f, (long long)mi * tiles_n + nt,
                            stage_block<BN>(o * tpr + mi, nt, kSub - 1, tiles_n) + kEpiBufBytes, err)) {
          ok = false;
          break;
        }
        const uint32_t* fl = f.red_ptrs[f.rank] + (size_t)o * f.flags_per_src + mi * tiles_n + nt;
        if (!wait_flag_ge(fl, f.epoch, abort_flag)) { ok = false; break; }
        fence_proxy_async_all();
        const int mt = o * tpr + mi;
        for (int sub = 0; sub < kSub; ++sub, ++item) {
          const uint32_t st = item % kCommStages;
          if (!mbar_wait(&cs->empty[st], ((item / kCommStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
          cs->meta[st] = ((((o * owned) + mi * tiles_n + nt) * kSub + sub) << 1) | 1;
          mbar_expect_tx(&cs->full[st], kEpiBufBytes);
          bulk_load(smem + st * kCommChunkBytes,
                    reinterpret_cast<const uint8_t*>(f.data_ptrs[o]) + stage_block<BN>(mt, nt, sub, tiles_n),
                    kEpiBufBytes, &cs->full[st]);
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
    const size_t y_row0 = all_reduce ? (size_t)f.rank * f.rows_per_rank : 0;
    uint8_t* own_stage = reinterpret_cast<uint8_t*>(f.data_ptrs[f.rank]);
    for (uint32_t item = 0;; ++item) {
      const uint32_t st = item % kCommStages;
      if (!mbar_wait(&cs->full[st], (item / kCommStages) & 1, abort_flag)) break;
      int code = cs->meta[st];
      if (code < 0) break;
      const bool last = (code >> 30) & 1;
      code &= ~(1 << 30);
      const uint8_t* base = smem + st * kCommChunkBytes;
      if ((code & 1) == 0) {
        code >>= 1;
        const int p = code % parts; code /= parts;
        const int sub = code % kSub; code /= kSub;
        const int nt = code % tiles_n, mi = code / tiles_n;
        const size_t blk = stage_block<BN>(f.rank * tpr + mi, nt, sub, tiles_n) + (size_t)p * src_bytes;
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
          const bf16x8 v = pack8(acc);
          if (col < N) *reinterpret_cast<bf16x8*>(f.y_local + (y_row0 + (size_t)mi * kBM + row) * N + col) = v;
          // all-reduce: the sum replaces this rank's own partial in its staging buffer, where the peers fetch it
          if (all_reduce) *reinterpret_cast<bf16x8*>(own_stage + blk + (size_t)q * 16) = v;
        }
        if (all_reduce && last) {
          named_bar_sync(2, kConsumers);      // every consumer's stores of this tile are issued
          if (ct == 0) {
            __threadfence_system();
            for (int d = 0; d < f.tp; ++d)
              if (d != f.rank)
                st_release_sys(f.red_ptrs[d] + (size_t)f.rank * f.flags_per_src + mi * tiles_n + nt, f.epoch);
          }
        }
      } else {
        code >>= 1;
        const int sub = code % kSub; code /= kSub;
        const int o = code / owned, tile = code % owned;
        const int nt = tile % tiles_n, mi = tile / tiles_n;
        for (int q = ct; q < kBM * 8; q += kConsumers) {
          const int row = q >> 3, cphys = q & 7;
          const int col = nt * BN + sub * 64 + ((cphys ^ (row & 7)) << 3);
          if (col < N)
            *reinterpret_cast<bf16x8*>(f.y_local + ((size_t)o * f.rows_per_rank + (size_t)mi * kBM + row) * N + col) =
                *reinterpret_cast<const bf16x8*>(base + q * 16);
        }
      }
      // the stage is refilled by a bulk load (async proxy): order this thread's generic-proxy reads before it
      fence_proxy_async_smem();
      mbar_arrive(&cs->empty[st]);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int old = atomicAdd(f.counter, 1u);
    if (old + 1 - f.counter_base == (unsigned int)nparts) {
      for (int p = 0; p < f.tp; ++p)
        if (p != f.rank) st_release_sys(f.done_ptrs[p] + f.rank, f.epoch);
    }
  }
}

// ---- tensor maps (gemm.cu) ----------------------------------------------------------------------------
int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                      uint32_t box_inner, uint32_t box_outer);
int make_tmap_f32_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                     uint32_t box_inner, uint32_t box_outer);
extern int g_no_tail_split;   // 1 keeps whole tiles in an under-filled last wave (ell_gemm_set_tail_split)
extern int g_rs_lag_q;        // see FuseArgs::rs_lag_q (ell_gemm_set_rs_lag)
extern unsigned long long g_fuse_data_bytes;   // size of every gathered / staging buffer (ell_gemm_set_fused_buffer_bytes)

}  // namespace ell
