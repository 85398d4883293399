// bf16 GEMM on CTA pairs: C[M,N] = op(A) · op(B)^T with one 256 x 256 output tile per two-CTA cluster.
//
// The two CTAs of a cluster sit on neighbouring SMs and run ONE tcgen05.mma.cta_group::2 stream, issued by a
// single thread of the even CTA ("leader").  Per 64-wide k-block each CTA stages only ITS half of the
// operands — 128 rows of A and 128 rows of B (16 KiB + 16 KiB) — and the tensor cores of both SMs read the
// two B halves from both shared memories.  Against the single-CTA kernel of gemm.cu (128 x 256 tile, 48 KiB
// per stage) that halves the shared-memory fill per FLOP and leaves room for six stages instead of four.
// Each CTA keeps the accumulator rows of its own A half in its own TMEM (128 lanes x 256 fp32 columns, two
// buffers) and runs its own epilogue on them.
//
// Synchronisation (every wait bounded, as in gemm.cu):
//   full[s]       in the leader only.  The leader's producer posts the byte count of BOTH CTAs' loads; the
//                 peer's loads complete on the leader's barrier (cp.async.bulk.tensor ... .cta_group::2 with
//                 the barrier address mapped into the leader's shared memory).
//   empty[s]      one per CTA; a tcgen05.commit that signals the same barrier offset in both CTAs tells both
//                 producers that the MMAs reading stage s are done.
//   tmem_full[a]  one per CTA, signalled the same way; tmem_empty[a] lives in the leader and collects the
//                 256 epilogue threads of both CTAs (the peer's threads arrive through the cluster address).
// Before a CTA leaves, its producer waits until the last commits on its own empty barriers have landed and
// the cluster meets at a cluster barrier, so nothing signals into the shared memory of a CTA that has exited.
//
// The same kernel carries the tensor-parallel fusions of gemm_fuse.cuh (all-gather -> GEMM on the A rows or on
// the reduction rows, GEMM -> reduce-scatter / all-reduce) and the cross-entropy epilogue of the LM head.  In a
// fused launch CTAs [0, n_comm) (whole clusters: n_comm is even) run the communication role; each CTA of a GEMM
// pair waits for the flag of its own 128 A rows.  Any M, N, K that the single-CTA kernel accepts (out-of-range
// parts of a tile are zero-filled on load and clipped on store); fused launches need rows_per_rank % 256 == 0.
//
// GEMM -> reduce-scatter here sums in the EPILOGUE, without a separate reduction pass: a tile that another rank
// owns is written (bf16, bulk stores through peer pointers) straight into that rank's staging buffer and flagged
// there; a tile this rank owns is computed `lag` rounds after the peers computed theirs, a seventh warp prefetches
// the peers' partial sums from the LOCAL staging buffer into the two epilogue buffers, and the epilogue adds them
// to the fp32 accumulator in a fixed source order before the one rounding to bf16 (deterministic; the own partial
// is never rounded).  GEMM -> all-reduce keeps the staged two-phase reduction of gemm_fuse.cuh.
#include "gemm_fuse.cuh"

namespace ell {
namespace pair {

constexpr int kTileM = 256, kTileN = 256;   // per cluster
constexpr int kHalfM = 128, kHalfN = 128;   // rows of A / rows of B staged by one CTA
constexpr int kThreads = kGemmThreads;      // warp 0 producer, warp 1 MMA issuer + TMEM owner, warps 2-5 epilogue
constexpr int kThreadsRS = kGemmThreads + 64;   // reduce-scatter form: warp 6 prefetches the peers' partial sums,
                                                // warp 7 sends staged blocks to their owners and raises the flags
constexpr int kStages = 6;
constexpr int kABytes = kHalfM * kBK * 2;   // 16 KiB
constexpr int kBBytes = kHalfN * kBK * 2;   // 16 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 2 * kTileN;       // two accumulator buffers
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kEpiBufBytes + 1024 + 512;
constexpr int kGroupM = 8;                  // rasterisation: 8 M-tiles x all N-tiles per group
enum Err { kErrPairProducer = 11, kErrPairMma = 12, kErrPairEpilogue = 13, kErrPairFlagWait = 15 };

struct Shared {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t part_full[2];    // reduce-scatter: a peer's partial 128 x 64 block has landed in epilogue buffer i
  uint64_t part_empty[2];   // ... and all 128 epilogue threads have added it
  uint64_t stage_free;      // ... the epilogue buffers are no longer read by bulk stores of staged blocks
  uint64_t chunk_ready[2];  // reduce-scatter: a staged 128 x 64 block sits in epilogue buffer i (128 writers)
  uint64_t buf_free[2];     // ... and the bulk store that sends it has read the buffer
  unsigned long long post_dst[2];   // where block i goes (a peer's staging buffer; 0: nowhere)
  unsigned long long post_flag[2];  // the flag to raise once the block and its predecessors of the tile have landed (0: none)
  uint32_t tmem_base;
  int abort_flag;
  int epi_abort;
};

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Address of `addr` (a shared-memory address of this CTA) inside CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Tile load into this CTA's shared memory whose completion bytes are counted on a barrier that may live in
// the other CTA of the pair (one destination CTA per copy).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "n"(kTmemCols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(kTmemCols) : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive on the barrier at this shared-memory offset in BOTH CTAs once every tcgen05.mma issued so far is done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(both)
               : "memory");
}

// __host__ __device__ so that the enumerate functions below can run the same code for a CPU coverage test
__host__ __device__ __forceinline__ void raster(int idx, int tiles_m, int tiles_n, int& mt, int& nt) {
  const int width = kGroupM * tiles_n;
  const int group = idx / width, rem = idx % width;
  const int first_m = group * kGroupM;
  const int gsz = (tiles_m - first_m) < kGroupM ? (tiles_m - first_m) : kGroupM;
  mt = first_m + rem % gsz;
  nt = rem / gsz;
}

// Work units of a launch.  When the last wave would leave at least half of the clusters idle, each of its tiles is
// cut into two half-width units (128 columns, tcgen05.mma with N = 128), so the tail costs half a wave:
// units [0, num_full) are whole tiles, unit num_full + 2i + h is half h of tile num_full + i.
struct Unit {
  int mt, nt, n0, bn;
  int kphase;   // kFuseAGK: which half of the (rotated) reduction range this unit accumulates
};

__host__ __device__ inline int split_tail(int num_tiles, int clusters, bool allowed) {
  const int tail = num_tiles % clusters;
  return (allowed && tail > 0 && 2 * tail <= clusters) ? tail : 0;
}

// Tile order of the fused forms (256-row tiles): all-gather -> GEMM walks the local shard's row tiles first and the
// other shards in ring order; GEMM -> reduce-scatter / all-reduce interleaves the owners so each is fed evenly.
// The gather of the reduction rows (kFuseAGK) walks every tile twice: first over the half of the k-range that
// starts at the local rows (while the peers' rows are still arriving), then over the other half; the output is an
// fp32 accumulation, so the two passes simply add up.
// Rounds by which a rank's own tiles trail the peers' in the reduce-scatter order: about two waves of tiles, so a
// partial sum has been computed, sent and flagged well before the owner's epilogue asks for it.
__host__ __device__ __forceinline__ int rs_lag(int tiles_per_owner, int n_clusters, int tp, int lag_q) {
  if (tp <= 1) return 0;
  const int q = lag_q > 0 ? lag_q : 8;                        // quarter waves; default two waves
  int lag = (q * n_clusters + 4 * tp - 1) / (4 * tp);
  if (lag < 1) lag = 1;
  return lag < tiles_per_owner ? lag : tiles_per_owner;
}

// Half-width units in the last wave of a reduce-scatter launch: only when every tile of that wave is one the rank
// owns (the closing `lag` tiles of its order are), because the peers' flags cover whole tiles.
__host__ __device__ __forceinline__ int rs_split_tail(int tiles_m, int tiles_n, int n_clusters, int tp, int lag_q,
                                                      bool allowed) {
  const int n = (tiles_m / (tp < 1 ? 1 : tp)) * tiles_n;
  const int tail = split_tail(tiles_m * tiles_n, n_clusters, allowed);
  return (tp <= 1 || tail <= rs_lag(n, n_clusters, tp, lag_q)) ? tail : 0;
}

// Reduce-scatter order of rank `rank`: round k computes tile k (raster order inside a shard) of every OTHER owner,
// nearest ring successor first, then the rank's own tile k - lag; the last `lag` own tiles close the launch.
// Returns the owner and sets `tile`.
__host__ __device__ __forceinline__ int rs_order(int pos, int n, int tp, int lag, int rank, int& tile) {
  const int head = lag * (tp - 1);
  if (pos < head) {
    tile = pos / (tp - 1);
    return (rank + 1 + pos % (tp - 1)) % tp;
  }
  pos -= head;
  if (pos < (n - lag) * tp) {
    const int k = lag + pos / tp, i = pos % tp;
    if (i < tp - 1) {
      tile = k;
      return (rank + 1 + i) % tp;
    }
    tile = k - lag;
    return rank;
  }
  tile = n - lag + (pos - (n - lag) * tp);
  return rank;
}

__host__ __device__ __forceinline__ Unit decode_unit(int unit, int tiles_m, int tiles_n, int num_full, int fuse, int rank,
                                                     int tp, int n_clusters, int lag_q = 0) {
  Unit u;
  int tile = unit, half = -1;
  if (unit >= num_full) {
    tile = num_full + ((unit - num_full) >> 1);
    half = (unit - num_full) & 1;
  }
  u.kphase = 0;
  if (fuse == kFuseAGK) {
    const int per_pass = tiles_m * tiles_n;
    u.kphase = tile / per_pass;
    tile -= u.kphase * per_pass;
  }
  if (fuse == kFuseAG) {
    const int tpr = tiles_m / tp, per_phase = tpr * tiles_n;
    const int phase = tile / per_phase;
    int mi;
    raster(tile % per_phase, tpr, tiles_n, mi, u.nt);
    u.mt = ((rank + phase) % tp) * tpr + mi;
  } else if (fuse == kFuseRS) {
    const int tpr = tiles_m / tp, n = tpr * tiles_n;
    int k, mi;
    const int owner = rs_order(tile, n, tp, rs_lag(n, n_clusters, tp, lag_q), rank, k);
    raster(k, tpr, tiles_n, mi, u.nt);
    u.mt = owner * tpr + mi;
  } else if (fuse == kFuseAR) {
    int mp;
    raster(tile, tiles_m, tiles_n, mp, u.nt);
    u.mt = (mp % tp) * (tiles_m / tp) + mp / tp;
  } else {
    raster(tile, tiles_m, tiles_n, u.mt, u.nt);
  }
  u.bn = half >= 0 ? kTileN / 2 : kTileN;
  u.n0 = u.nt * kTileN + (half > 0 ? kTileN / 2 : 0);
  return u;
}

// tmX: the local shard of the gathered operand (kFuseAG: A rows, box 128 x 64; kFuseAGK: reduction rows of B,
// box 64 x 64); tmBh: B with a box of 64 rows for the half-width units.
template <bool A_MN, bool B_MN, int OUT, bool HAS_BIAS, int FUSE>
__global__ void __launch_bounds__(FUSE == kFuseRS ? kThreadsRS : kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmBh,
                 const __grid_constant__ CUtensorMap tmX, const __grid_constant__ FuseArgs fuse,
                 const __grid_constant__ FuseArgs push, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                 int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr bool kReduce = (FUSE == kFuseRS || FUSE == kFuseAR);
  constexpr bool kGather = (FUSE == kFuseAG || FUSE == kFuseAGK);
  constexpr bool kStagedReduce = FUSE == kFuseAR;     // reduction as a separate role over staged tiles
  const int n_red = (FUSE == kFuseNone || FUSE == kFuseRS) ? 0 : fuse.n_comm;
  // reduce forms may carry the all-gather push of the next kernel's operand in CTAs [n_red, n_red + n_push)
  const int n_push = kReduce ? push.n_comm : 0;
  const int n_comm = n_red + n_push;                   // CTAs that do not run the GEMM
  const int tiles_m = (M + kTileM - 1) / kTileM, tiles_n = (N + kTileN - 1) / kTileN;

  if (FUSE != kFuseNone && (int)blockIdx.x < n_red) {
    // communication role; both CTAs of such a cluster take it, neither touches TMEM or the cluster barrier
    if (kGather) ag_comm_role(fuse, FUSE == kFuseAG ? K : N, err, smem, 0, n_red);
    else rs_reduce_role<kTileN>(fuse, N, tiles_n, err, smem, (int)gridDim.x - n_push, true, FUSE == kFuseAR);
    return;
  }
  if (kReduce && (int)blockIdx.x < n_comm) {
    ag_comm_role(push, push.shard_k, err, smem, n_red, n_push);
    return;
  }

  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * kABytes;
  uint8_t* sC = smem + kStages * kStageBytes;
  Shared* sh = reinterpret_cast<Shared*>(sC + 2 * kEpiBufBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_cta_rank();       // 0: leader, 1: peer
  const bool is_leader = cta_rank == 0;
  const int cluster_id = ((int)blockIdx.x - n_comm) >> 1, n_clusters = ((int)gridDim.x - n_comm) >> 1;
  const int k_passes = FUSE == kFuseAGK ? (fuse.k_passes == 2 ? 2 : 1) : 1;
  const int num_tiles = tiles_m * tiles_n * k_passes;   // kFuseAGK while the rows still arrive: two k-passes per tile
  const int num_kb = (K + kBK - 1) / kBK;
  const int n_split = FUSE == kFuseRS ? rs_split_tail(tiles_m, tiles_n, n_clusters, fuse.tp, fuse.rs_lag_q, !fuse.no_tail_split)
                                      : split_tail(num_tiles, n_clusters, !kReduce && !fuse.no_tail_split);
  const int num_full = num_tiles - n_split, num_units = num_tiles + n_split;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sh->tmem_full[a], 1);
      mbar_init(&sh->tmem_empty[a], 2 * kEpiThreads);
      mbar_init(&sh->part_full[a], 1);
      mbar_init(&sh->part_empty[a], kEpiThreads);
      mbar_init(&sh->chunk_ready[a], kEpiThreads);
      mbar_init(&sh->buf_free[a], 1);
    }
    mbar_init(&sh->stage_free, 1);
    sh->abort_flag = 0;
    sh->epi_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  __syncthreads();
  cluster_sync_all();                                  // both CTAs are resident and their barriers exist
  if (warp == 1) tmem_alloc_pair(&sh->tmem_base);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    // Two lanes share the issue work: lane 0 loads this CTA's A rows, lane 1 its B rows (the MN-major forms need
    // two 64-wide boxes per operand and k-block, and one thread issuing all four copies plus the barrier traffic
    // per 64-deep k-block was the slowest role of the weight-gradient GEMMs).  Both lanes walk the same units and
    // stages and wait on the same barriers; only the leader's lane 0 posts the expected byte count.
    if (lane < 2) {
      const bool loads_a = lane == 0;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // kFuseAGK: leading row tiles of every source rank already seen flagged (the k-loop revisits them per unit)
      int seen[kMaxTp];
#pragma unroll
      for (int i = 0; i < kMaxTp; ++i) seen[i] = 0;
      const int kpr = FUSE == kFuseAGK ? fuse.rows_per_rank / kBK : 1;   // k-blocks per source rank
      const int kb_rot = FUSE == kFuseAGK ? fuse.rank * kpr : 0;
      // one k-block: wait for the stage, post the byte count, issue this lane's copies
      auto load_kblock = [&](int kk, const CUtensorMap* a_map, int a_row, int m0, const CUtensorMap* b_map, int nb0,
                             int b_rows, int b_krow, uint32_t stage_tx) -> bool {
        if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) return false;
        if (is_leader && loads_a) mbar_expect_tx(&sh->full[stage], stage_tx);
        const uint32_t bar = map_to_cta(smem_u32(&sh->full[stage]), 0);
        // the same instruction stream for both lanes (selects, no divergent branches): a K-major operand is one
        // 64 x 128 box at (k, row), an MN-major operand one 64 x 64 box per 64 rows at (row + 64 i, k)
        const bool mn = loads_a ? A_MN : B_MN;
        uint8_t* dst = loads_a ? sA + stage * kABytes : sB + stage * kBBytes;
        const CUtensorMap* map = loads_a ? (A_MN ? &tmA : a_map) : b_map;
        const int row = loads_a ? (A_MN ? m0 : a_row) : nb0;
        const int kcoord = loads_a ? kk * kBK : (B_MN ? b_krow : kk * kBK);
        const int n_box = mn ? (loads_a ? kHalfM / 64 : b_rows / 64) : 1;
        for (int i = 0; i < n_box; ++i)
          tma_load_2d_pair(dst + i * (64 * kBK * 2), map, bar, mn ? row + i * 64 : kcoord, mn ? kcoord : row);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
        return true;
      };
      for (int unit = cluster_id; unit < num_units && ok; unit += n_clusters) {
        const Unit u = decode_unit(unit, tiles_m, tiles_n, num_full, FUSE, fuse.rank, fuse.tp, n_clusters, fuse.rs_lag_q);
        const int b_rows = u.bn / 2;                                // B rows staged by one CTA (128, or 64 in a half unit)
        const int m0 = u.mt * kTileM + (int)cta_rank * kHalfM;     // A rows of this CTA
        const int nb0 = u.n0 + (int)cta_rank * b_rows;             // B rows of this CTA
        const CUtensorMap* b_map = (u.bn == kTileN) ? &tmB : &tmBh; // half units: box of 64 B rows
        const uint32_t stage_tx = 2u * (kABytes + (uint32_t)b_rows * kBK * 2);
        const CUtensorMap* a_map = &tmA;
        int a_row = m0;
        if (FUSE == kFuseAG) {
          // the 128 A rows of this CTA come from rank `src`: the local shard is read in place, a remote shard
          // from the local gathered buffer once the peer's copy of this row tile is flagged
          const int src = m0 / fuse.rows_per_rank;
          if (src == fuse.rank) {
            a_map = &tmX;
            a_row = m0 - src * fuse.rows_per_rank;
          } else if (m0 < M) {
            const uint32_t* fl = fuse.flag_ptrs[fuse.rank] + (size_t)src * fuse.flags_per_src +
                                 (m0 - src * fuse.rows_per_rank) / kBM;
            if (!wait_flag_ge(fl, fuse.epoch, abort_flag)) {
              ok = false;
              atomicCAS(err, 0, kErrPairFlagWait);
              break;
            }
            fence_proxy_async_all();   // peer writes -> TMA reads (async proxy)
          }
        }
        if (FUSE != kFuseAGK) {
          for (int kb = 0; kb < num_kb && ok; ++kb)
            ok = load_kblock(kb, a_map, a_row, m0, b_map, nb0, b_rows, kb * kBK, stage_tx);
          continue;
        }
        // kFuseAGK: the k-range of this unit in rotated order (position r is k-block (r + kb_rot) mod num_kb, so the
        // walk starts at this rank's own rows), cut into runs that stay inside one source rank's rows: everything
        // that depends on the source is computed once per run, not once per k-block.
        int r = k_passes == 2 ? u.kphase * (num_kb / 2) : 0;
        const int r_hi = k_passes == 2 && u.kphase == 0 ? num_kb / 2 : num_kb;
        while (r < r_hi && ok) {
          int kk = r + kb_rot;
          if (kk >= num_kb) kk -= num_kb;
          const int src = kk / kpr;
          const int k_in = kk - src * kpr;                           // k-block inside the source's shard
          const int run = min(kpr - k_in, r_hi - r);
          const bool local = src == fuse.rank;
          const CUtensorMap* bk_map = local ? &tmX : &tmB;          // own rows in place, the others from the gathered buffer
          const int row0 = local ? 0 : src * fuse.rows_per_rank;
          int seen_src = seen[src];
          const uint32_t* flags = fuse.flag_ptrs[fuse.rank] + (size_t)src * fuse.flags_per_src;
          for (int i = 0; i < run && ok; ++i) {
            const int ki = k_in + i, tile = ki >> 1;                 // two 64-row k-blocks per flagged 128-row tile
            if (!local && tile >= seen_src) {
              if (!wait_flag_ge(flags + tile, fuse.epoch, abort_flag)) {
                ok = false;
                atomicCAS(err, 0, kErrPairFlagWait);
                break;
              }
              fence_proxy_async_all();
              seen_src = tile + 1;
            }
            ok = load_kblock(kk + i, a_map, a_row, m0, bk_map, nb0, b_rows, row0 + ki * kBK, stage_tx);
          }
          seen[src] = seen_src;
          r += run;
        }
      }
      // the leader's last commits on this CTA's empty barriers must have landed before the CTA may exit
      for (int s = 0; s < kStages && ok; ++s) {
        if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) ok = false;
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) {
        sh->abort_flag = 1;
        atomicCAS(err, 0, kErrPairProducer);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) --------------------------
    if (lane == 0 && is_leader) {
      constexpr uint32_t idesc_full = make_idesc_bf16(kTileM, kTileN, A_MN, B_MN);
      constexpr uint32_t idesc_half = make_idesc_bf16(kTileM, kTileN / 2, A_MN, B_MN);
      constexpr uint32_t a_lbo = A_MN ? 64 * kBK * 2 : 16, a_sbo = 1024, a_kstep = A_MN ? 2048 : 32;
      constexpr uint32_t b_lbo = B_MN ? 64 * kBK * 2 : 16, b_sbo = 1024, b_kstep = B_MN ? 2048 : 32;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int unit = cluster_id; unit < num_units && ok; unit += n_clusters, ++it) {
        const uint32_t idesc = unit >= num_full ? idesc_half : idesc_full;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&sh->tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kTileN;
        int n_kb = num_kb;
        if (k_passes == 2) {
          const int kphase = (unit >= num_full ? num_full + ((unit - num_full) >> 1) : unit) / (tiles_m * tiles_n);
          n_kb = kphase == 0 ? num_kb / 2 : num_kb - num_kb / 2;
        }
        for (int kb = 0; kb < n_kb; ++kb) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * kABytes);
          const uint32_t b_addr = smem_u32(sB + stage * kBBytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = make_smem_desc(a_addr + k * a_kstep, a_lbo, a_sbo);
            const uint64_t db = make_smem_desc(b_addr + k * b_kstep, b_lbo, b_sbo);
            umma_bf16_pair(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma_commit_pair(&sh->empty[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit_pair(&sh->tmem_full[acc]);
      }
      if (!ok) {
        sh->abort_flag = 1;
        atomicCAS(err, 0, kErrPairMma);
      }
    }
  } else if (warp == 7) {
    // ------------------------------ sender of staged blocks (reduce-scatter form) ----------
    // One thread issues every bulk store into the peers' staging buffers and raises the tile flags, so no epilogue
    // thread ever waits for a transfer over NVLink to complete or for a system-scope fence.
    if (FUSE == kFuseRS && lane == 0 && fuse.tp > 1) {
      bool ok = true;
      uint32_t sent = 0, freed = 0;
      auto release_read = [&](uint32_t upto) {      // buffers of blocks [freed, upto) have been read by their stores
        for (; freed < upto; ++freed) mbar_arrive(&sh->buf_free[freed & 1]);
      };
      for (int unit = cluster_id; unit < num_units && ok; unit += n_clusters) {
        const Unit u = decode_unit(unit, tiles_m, tiles_n, num_full, FUSE, fuse.rank, fuse.tp, n_clusters, fuse.rs_lag_q);
        if ((u.mt * kTileM) / fuse.rows_per_rank == fuse.rank) continue;
        for (int j = 0; j < u.bn / 64 && ok; ++j) {
          const uint32_t b = sent & 1;
          if (!mbar_wait(&sh->chunk_ready[b], (sent >> 1) & 1, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* dst = reinterpret_cast<uint8_t*>(sh->post_dst[b]);
          uint32_t* flag = reinterpret_cast<uint32_t*>(sh->post_flag[b]);
          if (dst != nullptr) bulk_store(dst, sC + b * kEpiBufBytes, kEpiBufBytes);
          tma_store_commit();
          ++sent;
          if (flag == nullptr) {
            tma_store_wait_read<1>();               // the store before this one has read its buffer
            release_read(sent - 1);
          } else {
            tma_store_wait_read<0>();
            release_read(sent);
            tma_store_wait_all<0>();                // the whole tile has landed on its owner
            fence_proxy_async_all();
            __threadfence_system();
            st_release_sys(flag, fuse.epoch);
          }
        }
      }
      tma_store_wait_all<0>();
      if (!ok) {
        sh->abort_flag = 1;
        atomicCAS(err, 0, kErrPairEpilogue);
      }
    }
  } else if (warp == 6) {
    // ------------------------------ partial-sum prefetch (reduce-scatter form) -------------
    // For every tile this rank owns: wait until all peers have flagged their partial block, then stream the
    // (tp - 1) x 4 staged 128 x 64 blocks from the LOCAL staging buffer through the two epilogue buffers, in the
    // order the epilogue adds them.
    if (FUSE == kFuseRS && lane == 0 && fuse.tp > 1) {
      const int tpr = fuse.rows_per_rank / kBM;
      bool ok = true;
      uint32_t item = 0, own_idx = 0;
      for (int unit = cluster_id; unit < num_units && ok; unit += n_clusters) {
        const Unit u = decode_unit(unit, tiles_m, tiles_n, num_full, FUSE, fuse.rank, fuse.tp, n_clusters, fuse.rs_lag_q);
        const int m0 = u.mt * kTileM + (int)cta_rank * kHalfM;
        if (m0 / fuse.rows_per_rank != fuse.rank) continue;
        const int mi = (m0 - fuse.rank * fuse.rows_per_rank) / kBM;
        const long long fidx = (long long)mi * tiles_n + u.nt;
        if (ok && !fuse_in_bounds(fuse, fidx,
                                  stage_block<kTileN>((fuse.tp - 1) * tpr + mi, u.nt, kTileN / 64 - 1, tiles_n) + kEpiBufBytes,
                                  err))
          ok = false;
        for (int si = 1; si < fuse.tp && ok; ++si) {
          const int src = (fuse.rank + si) % fuse.tp;
          ok = wait_flag_ge(fuse.flag_ptrs[fuse.rank] + (size_t)src * fuse.flags_per_src + fidx, fuse.epoch, abort_flag);
        }
        // the epilogue buffers stage the blocks of other owners' tiles in between: they are handed over when the
        // epilogue reaches this tile (the flags above, the long wait, have been taken ahead of it)
        if (ok) ok = mbar_wait(&sh->stage_free, own_idx & 1, abort_flag);
        ++own_idx;
        if (!ok) break;
        fence_proxy_async_all();       // peers' writes -> bulk loads (async proxy)
        const int j0 = (u.n0 - u.nt * kTileN) / 64;      // a half-width unit covers chunks 0-1 or 2-3 of its tile
        for (int j = j0; j < j0 + u.bn / 64 && ok; ++j)
          for (int si = 1; si < fuse.tp; ++si, ++item) {
            const int src = (fuse.rank + si) % fuse.tp;
            const uint32_t slot = item & 1;
            if (!mbar_wait(&sh->part_empty[slot], ((item >> 1) & 1) ^ 1, abort_flag)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&sh->part_full[slot], kEpiBufBytes);
            bulk_load(sC + slot * kEpiBufBytes,
                      reinterpret_cast<const uint8_t*>(fuse.data_ptrs[fuse.rank]) +
                          stage_block<kTileN>(src * tpr + mi, u.nt, j, tiles_n),
                      kEpiBufBytes, &sh->part_full[slot]);
          }
      }
      if (!ok) {
        sh->abort_flag = 1;
        atomicCAS(err, 0, kErrPairFlagWait);
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs, own 128 rows) --------------------
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    const bool store_thread = (threadIdx.x == 64);
    const uint32_t empty_bar0 = map_to_cta(smem_u32(&sh->tmem_empty[0]), 0);
    const uint32_t empty_bar1 = map_to_cta(smem_u32(&sh->tmem_empty[1]), 0);
    int it = 0;
    uint32_t store_count = 0;
    uint32_t* pending_flag = nullptr;   // reduce forms: flag of the last staged block, raised once its stores completed
    uint32_t part_item = 0;             // reduce-scatter: partial blocks consumed so far (selects buffer and parity)
    uint32_t staged = 0;                // reduce-scatter: blocks handed to warp 7 so far
    if (kReduce && store_thread) {
      // peers must have finished reading last epoch's staged tiles before they are overwritten
      for (int p = 0; p < fuse.tp; ++p)
        if (p != fuse.rank && !wait_flag_ge(fuse.done_ptrs[fuse.rank] + p, fuse.epoch - 1, abort_flag)) {
          sh->epi_abort = 1;
          atomicCAS(err, 0, kErrPairFlagWait);
        }
    }
    for (int unit = cluster_id; unit < num_units; unit += n_clusters, ++it) {
      const Unit u = decode_unit(unit, tiles_m, tiles_n, num_full, FUSE, fuse.rank, fuse.tp, n_clusters, fuse.rs_lag_q);
      const int m0 = u.mt * kTileM + (int)cta_rank * kHalfM, n0 = u.n0;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag)) sh->epi_abort = 1;
      named_bar_sync(1, kEpiThreads);
      if (*(volatile int*)&sh->epi_abort) break;   // uniform across the 128 epilogue threads
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * kTileN;
      float ce_m = -INFINITY, ce_s = 0.f, ce_t = 0.f;
      int ce_tcol = -1;                          // target column inside this unit, if any
      if (OUT == kOutBf16CE) {
        const int row = m0 + row_in_tile;
        if (row < M) {
          const long long tc = fuse.ce_target[row] - fuse.ce_vocab_start - n0;
          if (tc >= 0 && tc < u.bn && tc + n0 < fuse.ce_valid) ce_tcol = (int)tc;
        }
      }
      const bool own_tile = FUSE == kFuseRS && m0 / fuse.rows_per_rank == fuse.rank;
      if (own_tile && fuse.tp > 1) {
        // A tile this rank owns: add the peers' partial sums (prefetched by warp 6) and write the output shard.
        if (store_thread) {
          // the epilogue buffers may still be read by warp 7's stores of the last two staged blocks: hand them to
          // warp 6 after that
          for (uint32_t d = 1; d <= 2 && d <= staged; ++d) {
            const uint32_t c = staged - d;
            if (!mbar_wait(&sh->buf_free[c & 1], (c >> 1) & 1, abort_flag)) {
              sh->epi_abort = 1;
              sh->abort_flag = 1;
            }
          }
          mbar_arrive(&sh->stage_free);
        }
        const int row0_local = m0 - fuse.rank * fuse.rows_per_rank;
#pragma unroll 1
        for (int j = 0; j < u.bn / 64; ++j) {
          uint32_t r[64];
          tmem_ld_32x32(t_row + j * 64, r);
          tmem_ld_32x32(t_row + j * 64 + 32, r + 32);
          tmem_ld_wait();
          for (int si = 1; si < fuse.tp; ++si, ++part_item) {
            const uint32_t slot = part_item & 1;
            if (!mbar_wait(&sh->part_full[slot], (part_item >> 1) & 1, abort_flag)) {
              sh->epi_abort = 1;
              sh->abort_flag = 1;
            }
            uint8_t* prow = sC + slot * kEpiBufBytes + row_in_tile * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              float t[8];
              unpack8(*reinterpret_cast<const bf16x8*>(prow + ((c ^ (row_in_tile & 7)) << 4)), t);
#pragma unroll
              for (int e = 0; e < 8; ++e) r[c * 8 + e] = __float_as_uint(__uint_as_float(r[c * 8 + e]) + t[e]);
            }
            if (si == fuse.tp - 1) {
              // last source: the sum replaces the partial block in place (every thread rewrites the 128 bytes it just
              // read) and leaves through a tensor store; the buffer goes back to warp 6 once that store has read it
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                float t[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) t[e] = __uint_as_float(r[c * 8 + e]);
                *reinterpret_cast<bf16x8*>(prow + ((c ^ (row_in_tile & 7)) << 4)) = pack8(t);
              }
              fence_proxy_async_smem();
              named_bar_sync(1, kEpiThreads);
              if (store_thread) {
                tma_store_2d(&tmC, sC + slot * kEpiBufBytes, n0 + j * 64, row0_local);
                tma_store_commit();
                tma_store_wait_read<0>();
              }
              mbar_arrive(&sh->part_empty[slot]);
            } else {
              // The buffer goes back to warp 6, whose next bulk load (async proxy) overwrites it as soon as the 128th
              // arrive lands.  These reads went through the generic proxy: a proxy fence orders them before that write.
              fence_proxy_async_smem();
              mbar_arrive(&sh->part_empty[slot]);
            }
          }
        }
      } else if (OUT == kOutBf16 || OUT == kOutBf16CE) {
        // reduce-scatter, a tile another rank owns: the blocks go to warp 7 instead of being stored from here
        const bool to_sender = FUSE == kFuseRS && !own_tile;
#pragma unroll 1
        for (int j = 0; j < u.bn / 64; ++j) {
          uint8_t* buf = sC + ((to_sender ? staged : store_count) & 1) * kEpiBufBytes;
          if (to_sender) {
            if (!mbar_wait(&sh->buf_free[staged & 1], ((staged >> 1) & 1) ^ 1, abort_flag)) {
              sh->epi_abort = 1;
              sh->abort_flag = 1;
            }
          } else {
            if (store_thread) tma_store_wait_read<1>();
            named_bar_sync(1, kEpiThreads);
          }
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
          if (to_sender) {
            if (store_thread) {
              // the owner's staging buffer, slot of this source rank; the tile's last block carries its flag
              const int owner = m0 / fuse.rows_per_rank;
              const int mi = (m0 - owner * fuse.rows_per_rank) / kBM;
              const size_t off = stage_block<kTileN>(fuse.rank * (fuse.rows_per_rank / kBM) + mi, u.nt, j, tiles_n);
              const long long fidx = (long long)mi * tiles_n + u.nt;
              const bool ok_idx = fuse_in_bounds(fuse, fidx, off + kEpiBufBytes, err);
              sh->post_dst[staged & 1] =
                  ok_idx ? reinterpret_cast<unsigned long long>(reinterpret_cast<uint8_t*>(fuse.data_ptrs[owner]) + off) : 0ull;
              sh->post_flag[staged & 1] =
                  (ok_idx && j == u.bn / 64 - 1)
                      ? reinterpret_cast<unsigned long long>(fuse.flag_ptrs[owner] + (size_t)fuse.rank * fuse.flags_per_src + fidx)
                      : 0ull;
            }
            mbar_arrive(&sh->chunk_ready[staged & 1]);
            ++staged;
            continue;
          }
          named_bar_sync(1, kEpiThreads);
          if (store_thread) {
            if (own_tile) {
              // one-rank group: nothing to add, the tile is the output
              tma_store_2d(&tmC, buf, n0 + j * 64, m0 - fuse.rank * fuse.rows_per_rank);
            } else if (kReduce) {
              const size_t off = stage_block<kTileN>(m0 / kBM, u.nt, j, tiles_n);
              if (fuse_in_bounds(fuse, 0, off + kEpiBufBytes, err))
                bulk_store(reinterpret_cast<uint8_t*>(fuse.data_ptrs[fuse.rank]) + off, buf, kEpiBufBytes);
            } else if (n0 + j * 64 < N && m0 < M) {
              tma_store_2d(&tmC, buf, n0 + j * 64, m0);
            }
            tma_store_commit();
          }
          ++store_count;
        }
        if (OUT == kOutBf16CE) {
          // one slot of partials per 128 columns: a whole unit fills its first slot and neutralises the second
          const int row = m0 + row_in_tile;
          if (row < M) {
            float* part = fuse.ce_part + (size_t)(n0 / (kTileN / 2)) * 3 * M + row;
            part[0] = ce_m;
            part[(size_t)M] = ce_s;
            part[(size_t)2 * M] = ce_t;
            if (u.bn == kTileN) {
              part += (size_t)3 * M;
              part[0] = -INFINITY;
              part[(size_t)M] = 0.f;
              part[(size_t)2 * M] = 0.f;
            }
          }
        }
        if (kStagedReduce && store_thread) {
          // Publish the flag of the PREVIOUS block: its bulk stores were committed 4 groups ago, so waiting until
          // at most 4 groups are pending does not stall behind this block's stores.
          if (pending_flag != nullptr) {
            tma_store_wait_all<kTileN / 64>();
            fence_proxy_async_all();
            st_release_sys(pending_flag, fuse.epoch);
          }
          const int owner = m0 / fuse.rows_per_rank;
          const int mi = (m0 - owner * fuse.rows_per_rank) / kBM;
          pending_flag = fuse.flag_ptrs[owner] + (size_t)fuse.rank * fuse.flags_per_src + mi * tiles_n + u.nt;
        }
      } else {
        // fp32 output: 128 x 32 sub-tiles, stored or added into C at L2 by the TMA unit
#pragma unroll 1
        for (int j = 0; j < u.bn / 32; ++j) {
          uint8_t* buf = sC + (store_count & 1) * kEpiBufBytes;
          if (store_thread) tma_store_wait_read<1>();
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
          if (store_thread) {
            if (n0 + j * 32 < N && m0 < M) {
              if (OUT == kOutF32Accum) tma_reduce_add_2d(&tmC, buf, n0 + j * 32, m0);
              else tma_store_2d(&tmC, buf, n0 + j * 32, m0);
            }
            tma_store_commit();
          }
          ++store_count;
        }
      }
      tc_fence_before();
      mbar_arrive_cluster(acc ? empty_bar1 : empty_bar0);
    }
    if (*(volatile int*)&sh->epi_abort && store_thread) {
      sh->abort_flag = 1;
      atomicCAS(err, 0, kErrPairEpilogue);
    }
    if (store_thread) {
      tma_store_wait_all<0>();
      if (kStagedReduce && pending_flag != nullptr) {
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
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // neither CTA frees TMEM or exits while the other may still signal or read it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base);
  }
  if (kStagedReduce) {
    // the main loop is done: this CTA now helps summing the staged tiles its rank owns (the dedicated CTAs
    // [0, n_comm) have been doing so since launch)
    __syncthreads();
    rs_reduce_role<kTileN>(fuse, N, tiles_n, err, smem, (int)gridDim.x - n_push, true, FUSE == kFuseAR);
  }
  if ((kGather || FUSE == kFuseRS) && threadIdx.x == 0) {
    // last GEMM CTA of this rank: tell every peer that its pushes (gathered rows, or partial sums) of this epoch
    // were consumed
    __threadfence();
    const unsigned int old = atomicAdd(fuse.counter, 1u);
    if (old + 1 - fuse.counter_base == gridDim.x - (unsigned int)n_comm) {
      for (int p = 0; p < fuse.tp; ++p)
        if (p != fuse.rank) st_release_sys(fuse.done_ptrs[p] + fuse.rank, fuse.epoch);
    }
  }
}

// Clusters of a plain launch: every resident cluster when there is at least a wave of tiles; with less than half a
// wave, twice the tile count, so that every tile runs as two half-width units on two clusters.
__host__ inline int launch_clusters(int tiles, int resident) {
  if (tiles >= resident) return resident;
  if (!g_no_tail_split && 2 * tiles <= resident) return 2 * tiles;
  return tiles;
}

static int max_clusters(const void* kern) {
  static int n = 0;
  if (!n) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kNumSMs, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int c = 0;
    if (cudaOccupancyMaxActiveClusters(&c, kern, &cfg) != cudaSuccess || c <= 0) {
      cudaGetLastError();
      c = -1;
    }
    n = c;
  }
  return n;
}

// Fused launches keep a fixed grid (every resident cluster): the counters of the flag protocol count CTAs.
template <bool A_MN, bool B_MN, int OUT, bool HAS_BIAS, int FUSE = kFuseNone>
static int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC, const CUtensorMap& tBh,
                  const CUtensorMap& tX, const FuseArgs& fuse, const __nv_bfloat16* bias, int M, int N, int K, int* err,
                  cudaStream_t stream, const FuseArgs* push = nullptr) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, OUT, HAS_BIAS, FUSE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int resident = max_clusters(reinterpret_cast<const void*>(kern));
  if (resident <= 0) return -20;                 // the device cannot co-schedule a pair with this much shared memory
  const int tiles = ((M + kTileM - 1) / kTileM) * ((N + kTileN - 1) / kTileN);
  int grid;
  if (FUSE == kFuseNone) {
    grid = 2 * launch_clusters(tiles, resident);
  } else {
    const int n_role = fuse.n_comm + (push ? push->n_comm : 0);
    if ((fuse.n_comm & 1) || (n_role & 1) || n_role >= 2 * resident) return -2;
    grid = 2 * resident;
  }
  FuseArgs no_push{};
  const FuseArgs& push_args = push ? *push : no_push;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(FUSE == kFuseRS ? kThreadsRS : kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tA, tB, tC, tBh, tX, fuse, push_args, bias, M, N, K, err);
  if (e != cudaSuccess) {
    cudaGetLastError();   // a refused launch is reported to the caller, not left behind for the next launch
    return (int)e;
  }
  return launch_status();
}

static int resident_clusters() {
  auto kern = gemm_pair_kernel<false, false, kOutBf16, false, kFuseNone>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return max_clusters(reinterpret_cast<const void*>(kern));
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
  f.no_tail_split = g_no_tail_split;
  f.data_bytes = g_fuse_data_bytes;
  f.rs_lag_q = g_rs_lag_q;
}

// LM-head form: logits + cross-entropy partials, optionally behind the all-gather of the hidden rows.
static int gemm_ce(const void* X, const void* W, void* logits, const long long* target, float* part, int M, int N,
                   int K, long long vocab_start, int valid_cols, const FuseArgs* ag, const void* x_local, int* err,
                   cudaStream_t stream) {
  CUtensorMap tA, tB, tC, tBh, tX;
  int rc = make_tmap_bf16_2d(&tA, X, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kBK, kHalfM);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tB, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, kBK, kHalfN);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tBh, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, kBK, kHalfN / 2);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tC, logits, (uint64_t)N, (uint64_t)M, (uint64_t)N * 2, 64, 128);
  if (rc) return rc;
  tX = tA;
  FuseArgs f{};
  if (ag) {
    f = *ag;
    rc = make_tmap_bf16_2d(&tX, x_local, (uint64_t)K, (uint64_t)f.rows_per_rank, (uint64_t)K * 2, kBK, kHalfM);
    if (rc) return rc;
  }
  f.no_tail_split = g_no_tail_split;
  f.ce_target = target;
  f.ce_part = part;
  f.ce_vocab_start = vocab_start;
  f.ce_valid = valid_cols < N ? valid_cols : N;
  if (ag) return launch<false, false, kOutBf16CE, false, kFuseAG>(tA, tB, tC, tBh, tX, f, nullptr, M, N, K, err, stream);
  return launch<false, false, kOutBf16CE, false, kFuseNone>(tA, tB, tC, tBh, tX, f, nullptr, M, N, K, err, stream);
}

}  // namespace pair
}  // namespace ell

using namespace ell;

// Host-only: the 256 x 256 tiles of a launch in the order the clusters walk them (tile t goes to cluster
// t % clusters), from the kernel's own raster code.  out[t] = {row tile, column tile}.  Returns the tile count or -1.
ELL_API int ell_gemm_pair_enumerate_tiles(int M, int N, int* out, int max_tiles) {
  using namespace ell::pair;
  const int tiles_m = (M + kTileM - 1) / kTileM, tiles_n = (N + kTileN - 1) / kTileN;
  if (tiles_m * tiles_n > max_tiles) return -1;
  for (int t = 0; t < tiles_m * tiles_n; ++t) raster(t, tiles_m, tiles_n, out[2 * t], out[2 * t + 1]);
  return tiles_m * tiles_n;
}

// Host-only: the work units of a launch on `clusters` GEMM clusters in the order the kernel walks them (unit u goes to
// cluster u % clusters), tail halving included.  fuse: 0 plain, 1 all-gather -> GEMM, 2 GEMM -> reduce-scatter,
// 3 GEMM -> all-reduce, 4 all-gather of the reduction rows.  out[u] = {row tile, column tile, first column, width}.
// Returns the unit count or -1 when out is too small.
ELL_API int ell_gemm_pair_enumerate_units(int M, int N, int clusters, int allow_split, int fuse, int tp, int rank,
                                          int* out, int max_units) {
  using namespace ell::pair;
  const int tiles_m = (M + kTileM - 1) / kTileM, tiles_n = (N + kTileN - 1) / kTileN;
  const int num_tiles = tiles_m * tiles_n * (fuse == kFuseAGK ? 2 : 1);
  const bool reduce = fuse == kFuseRS || fuse == kFuseAR;
  const int n_split = fuse == kFuseRS ? rs_split_tail(tiles_m, tiles_n, clusters, tp < 1 ? 1 : tp, g_rs_lag_q, allow_split != 0)
                                      : split_tail(num_tiles, clusters, allow_split != 0 && !reduce);
  const int num_full = num_tiles - n_split, num_units = num_tiles + n_split;
  if (num_units > max_units) return -1;
  for (int u = 0; u < num_units; ++u) {
    const Unit t = decode_unit(u, tiles_m, tiles_n, num_full, fuse, rank, tp < 1 ? 1 : tp, clusters, g_rs_lag_q);
    out[4 * u + 0] = t.mt;
    out[4 * u + 1] = t.nt;
    out[4 * u + 2] = t.n0;
    out[4 * u + 3] = t.bn;
  }
  return num_units;
}

// Host-only: the order in which the reduce role takes the 128-row tiles a rank owns (queue position -> {row tile
// inside the shard, column tile}).  pair = 1: tiles staged by the CTA-pair kernel, 0: by the single-CTA kernel.
ELL_API int ell_gemm_owned_tile_order(int rows_per_rank, int tiles_n, int tp, int pair, int* out, int max_tiles) {
  const int tpr = rows_per_rank / kBM;
  if (tpr * tiles_n > max_tiles) return -1;
  for (int j = 0; j < tpr * tiles_n; ++j) owned_tile_of(j, tpr, tiles_n, tp, pair != 0, out[2 * j], out[2 * j + 1]);
  return tpr * tiles_n;
}

// Two-CTA clusters of the pair kernel that fit on the current device at once (needs a GPU; <= 0 if it cannot run).
// Rounds by which a rank's own tiles trail the peers' in the CTA-pair reduce-scatter, in quarter waves (0: default).
ELL_API void ell_gemm_set_rs_lag(int quarter_waves) { ell::g_rs_lag_q = quarter_waves < 0 ? 0 : quarter_waves; }

ELL_API int ell_gemm_pair_resident_clusters() { return ell::pair::resident_clusters(); }

// Clusters the kernel would launch for `tiles` tiles when `resident` clusters fit on the device.
ELL_API int ell_gemm_pair_launch_clusters(int tiles, int resident) { return ell::pair::launch_clusters(tiles, resident); }

// Same contract as ell_gemm_bf16 (without a tile-width hint): C = op(A)·op(B)^T, a_mn / b_mn select MN-major
// storage, out_mode 0 bf16 C, 1 fp32 C += result, 2 fp32 C = result; bias only with out_mode 0.
ELL_API int ell_gemm_bf16_pair(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                               int ldb, int ldc, int a_mn, int b_mn, int out_mode, int* err, cudaStream_t stream) {
  using namespace ell::pair;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (bias && out_mode != kOutBf16) return -2;
  if (out_mode < 0 || out_mode > 2) return -2;
  CUtensorMap tA, tB, tC;
  int rc;
  if (!a_mn) rc = make_tmap_bf16_2d(&tA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, kBK, kHalfM);
  else       rc = make_tmap_bf16_2d(&tA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, kBK);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_bf16_2d(&tB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kBK, kHalfN);
  else       rc = make_tmap_bf16_2d(&tB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, kBK);
  if (rc) return rc;
  if (out_mode == kOutBf16) rc = make_tmap_bf16_2d(&tC, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64, 128);
  else                      rc = make_tmap_f32_2d(&tC, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 4, 32, 128);
  if (rc) return rc;
  // B map with a box of 64 rows: the half-width units of a split tail wave stage 64 B rows per CTA
  CUtensorMap tBh = tB;
  if (!b_mn) {
    rc = make_tmap_bf16_2d(&tBh, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kBK, kHalfN / 2);
    if (rc) return rc;
  }
  FuseArgs f{};
  f.no_tail_split = g_no_tail_split;
  const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(bias);
#define ELL_PAIR_CASE(AM_, BM_, OUT_, BIAS_)                                                   \
  if ((bool)a_mn == AM_ && (bool)b_mn == BM_ && out_mode == OUT_ && (bias != nullptr) == BIAS_) \
    return launch<AM_, BM_, OUT_, BIAS_>(tA, tB, tC, tBh, tA, f, bp, M, N, K, err, stream);
  ELL_PAIR_CASE(false, false, kOutBf16, false)
  ELL_PAIR_CASE(false, false, kOutBf16, true)
  ELL_PAIR_CASE(false, true, kOutBf16, false)
  ELL_PAIR_CASE(true, true, kOutBf16, false)
  ELL_PAIR_CASE(true, true, kOutF32Accum, false)
  ELL_PAIR_CASE(true, true, kOutF32, false)
  ELL_PAIR_CASE(false, false, kOutF32, false)
  ELL_PAIR_CASE(false, true, kOutF32, false)
#undef ELL_PAIR_CASE
  return -3;
}

// Slots of cross-entropy partials the CTA-pair epilogue fills (one per 128 columns).
ELL_API int ell_gemm_ce_slots_pair(int N) { return 2 * ((N + 255) / 256); }

// logits[M, N] (bf16) = X[M, K] · W[N, K]^T on CTA pairs with the cross-entropy statistics fused into the epilogue:
// part[slots][3][M] = (max, sum exp(x - max), logit of the target if it falls in the slot else 0) over the first
// `valid_cols` columns; target holds global vocabulary ids, column 0 is id vocab_start.
ELL_API int ell_gemm_ce_pair(const void* X, const void* W, void* logits, const long long* target, float* part, int M,
                             int N, int K, long long vocab_start, int valid_cols, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return ell::pair::gemm_ce(X, W, logits, target, part, M, N, K, vocab_start, valid_cols, nullptr, nullptr, err, stream);
}

// Total CTAs of a fused CTA-pair launch (communication CTAs included): the host advances its copy of the CTA
// counter by this (reduce forms) or by this minus n_comm (gather forms) per launch.
ELL_API int ell_gemm_pair_fused_grid() {
  const int r = ell::pair::resident_clusters();
  return r > 0 ? 2 * r : -1;
}

// All-gather -> GEMM on CTA pairs (contract of ell_gemm_ag; rows_per_rank % 256 == 0, n_comm even).  With
// ce_target != nullptr the epilogue also emits the cross-entropy partials of ell_gemm_ce_pair (LM head).
ELL_API int ell_gemm_ag_pair(const void* x_local, const void* W, void* out, const void* bias, int rows_per_rank, int N,
                             int K, int b_mn, int rank, int tp, unsigned int epoch, int n_comm,
                             void* const* gathered_ptrs, void* const* flag_ptrs, void* const* done_ptrs, void* counter,
                             unsigned int counter_base, int flags_per_src, const long long* ce_target, float* ce_part,
                             long long ce_vocab_start, int ce_valid, int* err, cudaStream_t stream) {
  using namespace ell::pair;
  if (tp < 1 || tp > kMaxTp || rows_per_rank % kTileM || rows_per_rank / kBM > flags_per_src) return -2;
  if (b_mn && (bias || ce_target)) return -2;
  if (n_comm < 2 || (n_comm & 1)) return -2;
  const int M = rows_per_rank * tp;
  FuseArgs f{};
  fill_fuse(f, rank, tp, n_comm, rows_per_rank, flags_per_src, epoch, gathered_ptrs, flag_ptrs, nullptr, done_ptrs,
            counter, counter_base);
  f.x_local = (const __nv_bfloat16*)x_local;
  if (ce_target) {
    if (bias) return -2;
    return gemm_ce(gathered_ptrs[rank], W, out, ce_target, ce_part, M, N, K, ce_vocab_start, ce_valid, &f, x_local, err,
                   stream);
  }
  CUtensorMap tA, tB, tC, tBh, tX;
  int rc = make_tmap_bf16_2d(&tA, gathered_ptrs[rank], (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kBK, kHalfM);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_bf16_2d(&tB, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, kBK, kHalfN);
  else       rc = make_tmap_bf16_2d(&tB, W, (uint64_t)N, (uint64_t)K, (uint64_t)N * 2, 64, kBK);
  if (rc) return rc;
  tBh = tB;
  if (!b_mn) {
    rc = make_tmap_bf16_2d(&tBh, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, kBK, kHalfN / 2);
    if (rc) return rc;
  }
  rc = make_tmap_bf16_2d(&tC, out, (uint64_t)N, (uint64_t)M, (uint64_t)N * 2, 64, 128);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tX, x_local, (uint64_t)K, (uint64_t)rows_per_rank, (uint64_t)K * 2, kBK, kHalfM);
  if (rc) return rc;
  const __nv_bfloat16* bp = (const __nv_bfloat16*)bias;
  if (b_mn) return launch<false, true, kOutBf16, false, kFuseAG>(tA, tB, tC, tBh, tX, f, bp, M, N, K, err, stream);
  if (bias) return launch<false, false, kOutBf16, true, kFuseAG>(tA, tB, tC, tBh, tX, f, bp, M, N, K, err, stream);
  return launch<false, false, kOutBf16, false, kFuseAG>(tA, tB, tC, tBh, tX, f, bp, M, N, K, err, stream);
}

// Weight gradient behind the all-gather of its reduction rows, on CTA pairs:
//   dW[Nout, Kin] (fp32) += dy[T, Nout]^T · gather(x_local)[T, Kin],   T = tp * rows_per_rank.
// The communication CTAs push this rank's x rows to the peers' gathered buffers; every output tile starts its k-loop
// on the local rows and waits for a remote row tile right before its first k-block.
ELL_API int ell_gemm_agk_wgrad_pair(const void* dy, const void* x_local, void* dW, int rows_per_rank, int Nout, int Kin,
                                    int rank, int tp, unsigned int epoch, int n_comm, void* const* gathered_ptrs,
                                    void* const* flag_ptrs, void* const* done_ptrs, void* counter,
                                    unsigned int counter_base, int flags_per_src, int* err, cudaStream_t stream) {
  using namespace ell::pair;
  if (tp < 1 || tp > kMaxTp || rows_per_rank % kTileM || rows_per_rank / kBM > flags_per_src) return -2;
  // n_comm = 0: the rows were pushed by an earlier launch of this epoch (ell_gemm_rs_pair with a push)
  if (n_comm < 0 || (n_comm & 1) || Nout % 8 || Kin % 8) return -2;
  const int T = rows_per_rank * tp;
  CUtensorMap tA, tB, tC, tX;
  int rc = make_tmap_bf16_2d(&tA, dy, (uint64_t)Nout, (uint64_t)T, (uint64_t)Nout * 2, 64, kBK);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tB, gathered_ptrs[rank], (uint64_t)Kin, (uint64_t)T, (uint64_t)Kin * 2, 64, kBK);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tX, x_local, (uint64_t)Kin, (uint64_t)rows_per_rank, (uint64_t)Kin * 2, 64, kBK);
  if (rc) return rc;
  rc = make_tmap_f32_2d(&tC, dW, (uint64_t)Kin, (uint64_t)Nout, (uint64_t)Kin * 4, 32, 128);
  if (rc) return rc;
  FuseArgs f{};
  fill_fuse(f, rank, tp, n_comm, rows_per_rank, flags_per_src, epoch, gathered_ptrs, flag_ptrs, nullptr, done_ptrs,
            counter, counter_base);
  f.x_local = (const __nv_bfloat16*)x_local;
  f.k_passes = n_comm > 0 ? 2 : 1;   // rows pushed by this launch arrive during the first pass over the local half
  return launch<true, true, kOutF32Accum, false, kFuseAGK>(tA, tB, tC, tB, tX, f, nullptr, Nout, Kin, T, err, stream);
}

// GEMM -> reduce-scatter (all_reduce = 0; contract of ell_gemm_rs) or GEMM -> all-reduce (all_reduce = 1: y is the
// full [tp * rows_per_rank, N] output and red_ptrs[r] rank r's "tile reduced" flags) on CTA pairs.
// rows_per_rank % 256 == 0, N % 256 == 0, n_comm even.
// push_x != nullptr: n_push more CTAs copy the shard push_x [push_rows, push_k] into the peers' gathered buffers
// (gathered_ptrs / ag_flag_ptrs / ag_done_ptrs, epoch push_epoch) for the kernel that follows on the stream
// (ell_gemm_agk_wgrad_pair with n_comm = 0 and the same epoch).
ELL_API int ell_gemm_rs_pair(const void* x, const void* W, void* y, int rows_per_rank, int N, int K, int b_mn, int rank,
                             int tp, unsigned int epoch, int n_comm, void* const* stage_ptrs, void* const* flag_ptrs,
                             void* const* red_ptrs, void* const* done_ptrs, void* counter, unsigned int counter_base,
                             int flags_per_src, unsigned int queue_base, int all_reduce, const void* push_x,
                             int push_rows, int push_k, unsigned int push_epoch, int n_push,
                             void* const* gathered_ptrs, void* const* ag_flag_ptrs, void* const* ag_done_ptrs, int* err,
                             cudaStream_t stream) {
  using namespace ell::pair;
  if (tp < 1 || tp > kMaxTp || rows_per_rank % kTileM || N % kTileN) return -2;
  if (n_comm & 1) return -2;
  if (all_reduce && !red_ptrs) return -2;
  const int M = rows_per_rank * tp;
  const int tiles_n = N / kTileN;
  if ((rows_per_rank / kBM) * tiles_n > flags_per_src) return -2;
  CUtensorMap tA, tB, tC;
  int rc = make_tmap_bf16_2d(&tA, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kBK, kHalfM);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_bf16_2d(&tB, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, kBK, kHalfN);
  else       rc = make_tmap_bf16_2d(&tB, W, (uint64_t)N, (uint64_t)K, (uint64_t)N * 2, 64, kBK);
  if (rc) return rc;
  // all-reduce stages whole tiles locally; reduce-scatter writes the tiles it owns straight into the output shard
  // B with a box of 64 rows for the half-width units that may close a reduce-scatter launch
  CUtensorMap tBh = tB;
  if (!b_mn) {
    rc = make_tmap_bf16_2d(&tBh, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, kBK, kHalfN / 2);
    if (rc) return rc;
  }
  if (all_reduce) rc = make_tmap_bf16_2d(&tC, stage_ptrs[rank], (uint64_t)N, (uint64_t)M, (uint64_t)N * 2, 64, 128);
  else            rc = make_tmap_bf16_2d(&tC, y, (uint64_t)N, (uint64_t)rows_per_rank, (uint64_t)N * 2, 64, 128);
  if (rc) return rc;
  FuseArgs f{};
  // the reduce-scatter form sums in its epilogue: no reduce CTAs, no tile queue
  fill_fuse(f, rank, tp, all_reduce ? n_comm : 0, rows_per_rank, flags_per_src, epoch, stage_ptrs, flag_ptrs, red_ptrs,
            done_ptrs, counter, counter_base);
  f.y_local = (__nv_bfloat16*)y;
  f.queue_base = queue_base;
  FuseArgs ps{};
  const FuseArgs* pp = nullptr;
  if (push_x != nullptr && n_push > 0) {
    if ((n_push & 1) || push_rows % kBM || push_rows / kBM > flags_per_src || push_k % 8) return -2;
    fill_fuse(ps, rank, tp, n_push, push_rows, flags_per_src, push_epoch, gathered_ptrs, ag_flag_ptrs, nullptr,
              ag_done_ptrs, counter, 0);
    ps.x_local = (const __nv_bfloat16*)push_x;
    ps.shard_k = push_k;
    pp = &ps;
  }
  if (all_reduce) {
    if (b_mn) return launch<false, true, kOutBf16, false, kFuseAR>(tA, tB, tC, tB, tA, f, nullptr, M, N, K, err, stream, pp);
    return launch<false, false, kOutBf16, false, kFuseAR>(tA, tB, tC, tB, tA, f, nullptr, M, N, K, err, stream, pp);
  }
  if (b_mn) return launch<false, true, kOutBf16, false, kFuseRS>(tA, tB, tC, tBh, tA, f, nullptr, M, N, K, err, stream, pp);
  return launch<false, false, kOutBf16, false, kFuseRS>(tA, tB, tC, tBh, tA, f, nullptr, M, N, K, err, stream, pp);
}
