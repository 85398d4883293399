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
// Restrictions: plain launches only (no collective fusion, no cross-entropy epilogue); any M, N, K that the
// single-CTA kernel accepts (out-of-range parts of a tile are zero-filled on load and clipped on store).
#include "common.cuh"
#include "sm100.cuh"

namespace ell {
using namespace sm100;

int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                      uint32_t box_inner, uint32_t box_outer);
int make_tmap_f32_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                     uint32_t box_inner, uint32_t box_outer);

extern int g_no_tail_split;   // gemm.cu: 1 keeps whole tiles in an under-filled last wave (ell_gemm_set_tail_split)

namespace pair {

constexpr int kTileM = 256, kTileN = 256;   // per cluster
constexpr int kHalfM = 128, kHalfN = 128;   // rows of A / rows of B staged by one CTA
constexpr int kBK = 64;
constexpr int kThreads = 192;               // warp 0 producer, warp 1 MMA issuer + TMEM owner, warps 2-5 epilogue
constexpr int kEpiThreads = 128;
constexpr int kStages = 6;
constexpr int kABytes = kHalfM * kBK * 2;   // 16 KiB
constexpr int kBBytes = kHalfN * kBK * 2;   // 16 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kEpiBufBytes = 128 * 64 * 2;
constexpr int kTmemCols = 2 * kTileN;       // two accumulator buffers
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kEpiBufBytes + 1024 + 256;
constexpr int kGroupM = 8;                  // rasterisation: 8 M-tiles x all N-tiles per group
enum Out { kOutBf16 = 0, kOutF32Accum = 1, kOutF32 = 2 };
enum Err { kErrProducer = 11, kErrMma = 12, kErrEpilogue = 13 };

struct Shared {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
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

// __host__ __device__ so that ell_gemm_pair_enumerate_tiles can run the same code for a CPU coverage test
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
};

__host__ __device__ inline int split_tail(int num_tiles, int clusters, bool allowed) {
  const int tail = num_tiles % clusters;
  return (allowed && tail > 0 && 2 * tail <= clusters) ? tail : 0;
}

__host__ __device__ __forceinline__ Unit decode_unit(int unit, int tiles_m, int tiles_n, int num_full) {
  Unit u;
  int tile = unit, half = -1;
  if (unit >= num_full) {
    tile = num_full + ((unit - num_full) >> 1);
    half = (unit - num_full) & 1;
  }
  raster(tile, tiles_m, tiles_n, u.mt, u.nt);
  u.bn = half >= 0 ? kTileN / 2 : kTileN;
  u.n0 = u.nt * kTileN + (half > 0 ? kTileN / 2 : 0);
  return u;
}

template <bool A_MN, bool B_MN, int OUT, bool HAS_BIAS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmBh,
                 const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int tail_split, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * kABytes;
  uint8_t* sC = smem + kStages * kStageBytes;
  Shared* sh = reinterpret_cast<Shared*>(sC + 2 * kEpiBufBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_cta_rank();       // 0: leader, 1: peer
  const bool is_leader = cta_rank == 0;
  const int cluster_id = (int)blockIdx.x >> 1, n_clusters = (int)gridDim.x >> 1;
  const int tiles_m = (M + kTileM - 1) / kTileM, tiles_n = (N + kTileN - 1) / kTileN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + kBK - 1) / kBK;
  const int n_split = split_tail(num_tiles, n_clusters, tail_split != 0);
  const int num_full = num_tiles - n_split, num_units = num_tiles + n_split;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sh->tmem_full[a], 1);
      mbar_init(&sh->tmem_empty[a], 2 * kEpiThreads);
    }
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
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = cluster_id; unit < num_units && ok; unit += n_clusters) {
        const Unit u = decode_unit(unit, tiles_m, tiles_n, num_full);
        const int b_rows = u.bn / 2;                                // B rows staged by one CTA (128, or 64 in a half unit)
        const int m0 = u.mt * kTileM + (int)cta_rank * kHalfM;     // A rows of this CTA
        const int nb0 = u.n0 + (int)cta_rank * b_rows;             // B rows of this CTA
        const CUtensorMap* b_map = (u.bn == kTileN) ? &tmB : &tmBh; // half units: box of 64 B rows
        const uint32_t stage_tx = 2u * (kABytes + (uint32_t)b_rows * kBK * 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          if (is_leader) mbar_expect_tx(&sh->full[stage], stage_tx);
          const uint32_t bar = map_to_cta(smem_u32(&sh->full[stage]), 0);
          uint8_t* a_dst = sA + stage * kABytes;
          uint8_t* b_dst = sB + stage * kBBytes;
          if (!A_MN) {
            tma_load_2d_pair(a_dst, &tmA, bar, kb * kBK, m0);
          } else {
#pragma unroll
            for (int i = 0; i < kHalfM / 64; ++i)
              tma_load_2d_pair(a_dst + i * (64 * kBK * 2), &tmA, bar, m0 + i * 64, kb * kBK);
          }
          if (!B_MN) {
            tma_load_2d_pair(b_dst, b_map, bar, kb * kBK, nb0);
          } else {
#pragma unroll
            for (int i = 0; i < kHalfN / 64; ++i)
              if (i * 64 < b_rows) tma_load_2d_pair(b_dst + i * (64 * kBK * 2), &tmB, bar, nb0 + i * 64, kb * kBK);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
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
        atomicCAS(err, 0, kErrProducer);
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
        for (int kb = 0; kb < num_kb; ++kb) {
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
        atomicCAS(err, 0, kErrMma);
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
    for (int unit = cluster_id; unit < num_units; unit += n_clusters, ++it) {
      const Unit u = decode_unit(unit, tiles_m, tiles_n, num_full);
      const int m0 = u.mt * kTileM + (int)cta_rank * kHalfM, n0 = u.n0;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag)) sh->epi_abort = 1;
      named_bar_sync(1, kEpiThreads);
      if (*(volatile int*)&sh->epi_abort) break;   // uniform across the 128 epilogue threads
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * kTileN;
      if (OUT == kOutBf16) {
#pragma unroll 1
        for (int j = 0; j < u.bn / 64; ++j) {
          uint8_t* buf = sC + (store_count & 1) * kEpiBufBytes;
          if (store_thread) tma_store_wait_read<1>();
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
          if (store_thread) {
            if (n0 + j * 64 < N && m0 < M) tma_store_2d(&tmC, buf, n0 + j * 64, m0);
            tma_store_commit();
          }
          ++store_count;
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
      atomicCAS(err, 0, kErrEpilogue);
    }
    if (store_thread) tma_store_wait_all<0>();
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
}

// Clusters of a launch: every resident cluster when there is at least a wave of tiles; with less than half a wave,
// twice the tile count, so that every tile runs as two half-width units on two clusters.
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

template <bool A_MN, bool B_MN, int OUT, bool HAS_BIAS>
static int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC, const CUtensorMap& tBh,
                  const __nv_bfloat16* bias, int M, int N, int K, int* err, cudaStream_t stream) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, OUT, HAS_BIAS>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int resident = max_clusters(reinterpret_cast<const void*>(kern));
  if (resident <= 0) return -20;                 // the device cannot co-schedule a pair with this much shared memory
  const int tiles = ((M + kTileM - 1) / kTileM) * ((N + kTileN - 1) / kTileN);
  const int clusters = launch_clusters(tiles, resident);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tA, tB, tC, tBh, bias, M, N, K, g_no_tail_split ? 0 : 1, err);
  if (e != cudaSuccess) {
    cudaGetLastError();   // a refused launch is reported to the caller, not left behind for the next launch
    return (int)e;
  }
  return launch_status();
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

// Host-only: the work units of a launch on `clusters` clusters in the order the kernel walks them (unit u goes to
// cluster u % clusters), tail halving included.  out[u] = {row tile, column tile, first column, width}.  Returns the
// unit count or -1 when out is too small.
ELL_API int ell_gemm_pair_enumerate_units(int M, int N, int clusters, int allow_split, int* out, int max_units) {
  using namespace ell::pair;
  const int tiles_m = (M + kTileM - 1) / kTileM, tiles_n = (N + kTileN - 1) / kTileN;
  const int num_tiles = tiles_m * tiles_n;
  const int n_split = split_tail(num_tiles, clusters, allow_split != 0);
  const int num_full = num_tiles - n_split, num_units = num_tiles + n_split;
  if (num_units > max_units) return -1;
  for (int u = 0; u < num_units; ++u) {
    const Unit t = decode_unit(u, tiles_m, tiles_n, num_full);
    out[4 * u + 0] = t.mt;
    out[4 * u + 1] = t.nt;
    out[4 * u + 2] = t.n0;
    out[4 * u + 3] = t.bn;
  }
  return num_units;
}

// Two-CTA clusters of the pair kernel that fit on the current device at once (needs a GPU; <= 0 if it cannot run).
ELL_API int ell_gemm_pair_resident_clusters() {
  using namespace ell::pair;
  auto kern = gemm_pair_kernel<false, false, kOutBf16, false>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return max_clusters(reinterpret_cast<const void*>(kern));
}

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
  const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(bias);
#define ELL_PAIR_CASE(AM_, BM_, OUT_, BIAS_)                                                   \
  if ((bool)a_mn == AM_ && (bool)b_mn == BM_ && out_mode == OUT_ && (bias != nullptr) == BIAS_) \
    return launch<AM_, BM_, OUT_, BIAS_>(tA, tB, tC, tBh, bp, M, N, K, err, stream);
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
