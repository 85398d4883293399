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

enum GemmOut { kOutBf16 = 0, kOutF32Accum = 1, kOutF32 = 2 };
enum GemmErr { kErrProducer = 1, kErrMma = 2, kErrEpilogue = 3 };

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

template <int BN, bool A_MN, bool B_MN, int OUT, bool HAS_BIAS>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, float* __restrict__ Cf32,
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
    if (OUT == kOutBf16) tma_prefetch_desc(&tmC);
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
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * kBM, n0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&sh->full[stage], Cfg::kStageBytes);
          uint8_t* a_dst = sA + stage * kABytes;
          uint8_t* b_dst = sB + stage * Cfg::kBBytes;
          if (!A_MN) {
            tma_load_2d(a_dst, &tmA, &sh->full[stage], kb * kBK, m0);
          } else {
#pragma unroll
            for (int i = 0; i < kBM / 64; ++i)
              tma_load_2d(a_dst + i * (64 * kBK * 2), &tmA, &sh->full[stage], m0 + i * 64, kb * kBK);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, &tmB, &sh->full[stage], kb * kBK, n0);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(b_dst + i * (64 * kBK * 2), &tmB, &sh->full[stage], n0 + i * 64, kb * kBK);
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
      constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, A_MN, B_MN);
      // K-major: 8-row groups 1024 B apart; one K=16 step is 32 B inside the swizzle row.
      // MN-major: 64-element MN groups one [64 x kBK] box (8 KiB) apart, 8-K groups 1024 B apart;
      // one K=16 step is two such groups (2 KiB).
      constexpr uint32_t a_lbo = A_MN ? 64 * kBK * 2 : 16, a_sbo = 1024, a_kstep = A_MN ? 2048 : 32;
      constexpr uint32_t b_lbo = B_MN ? 64 * kBK * 2 : 16, b_sbo = 1024, b_kstep = B_MN ? 2048 : 32;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
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
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int m0 = (tile % tiles_m) * kBM, n0 = (tile / tiles_m) * BN;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag)) sh->epi_abort = 1;
      named_bar_sync(1, kEpiThreads);
      if (*(volatile int*)&sh->epi_abort) break;   // uniform across the 128 epilogue threads
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      if (OUT == kOutBf16) {
#pragma unroll 1
        for (int j = 0; j < BN / 64; ++j) {
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
            if (n0 + j * 64 < N) tma_store_2d(&tmC, buf, n0 + j * 64, m0);
            tma_store_commit();
          }
          ++store_count;
        }
      } else {
        const int row = m0 + row_in_tile;
#pragma unroll 1
        for (int j = 0; j < BN / 32; ++j) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + j * 32, r);   // warp-collective: every lane participates
          tmem_ld_wait();
          const int col0 = n0 + j * 32;
          if (row < M && col0 < N) {
            float* dst = Cf32 + (size_t)row * ldc + col0;
            if (col0 + 32 <= N && (ldc & 3) == 0) {
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                float4 v = make_float4(__uint_as_float(r[4 * c]), __uint_as_float(r[4 * c + 1]),
                                       __uint_as_float(r[4 * c + 2]), __uint_as_float(r[4 * c + 3]));
                if (OUT == kOutF32Accum) {
                  float4 o = reinterpret_cast<float4*>(dst)[c];
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                reinterpret_cast<float4*>(dst)[c] = v;
              }
            } else {
              for (int c = 0; c < 32 && col0 + c < N; ++c) {
                float v = __uint_as_float(r[c]);
                if (OUT == kOutF32Accum) v += dst[c];
                dst[c] = v;
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&sh->tmem_empty[acc]);
    }
    if (*(volatile int*)&sh->epi_abort && leader) {
      sh->abort_flag = 1;
      atomicCAS(err, 0, kErrEpilogue);
    }
    if (OUT == kOutBf16 && leader) tma_store_wait_all<0>();
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
int make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                      uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -10;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (row_stride_bytes & 15)) return -11;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

template <int BN, bool A_MN, bool B_MN, int OUT, bool HAS_BIAS>
static int launch_gemm(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC, float* Cf32,
                       const __nv_bfloat16* bias, int M, int N, int K, int ldc, int* err, int max_ctas,
                       cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OUT, HAS_BIAS>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
  int grid = tiles < max_ctas ? tiles : max_ctas;
  kern<<<grid, kGemmThreads, GemmCfg<BN>::kSmemBytes, stream>>>(tA, tB, tC, Cf32, bias, M, N, K, ldc, err);
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

// C = op(A)·op(B)^T.  a_mn / b_mn select MN-major storage ([K,M] / [K,N] row-major).
// out_mode: 0 bf16 C (ldc in elements), 1 fp32 C += result, 2 fp32 C = result.
// `err` is a device int that receives a non-zero code if a bounded wait inside the kernel expired.
ELL_API int ell_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                          int ldb, int ldc, int a_mn, int b_mn, int out_mode, int bn_hint, int* err,
                          cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (bias && out_mode != kOutBf16) return -2;
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
    tC = tA;
  }
  const int ctas = sm_count();
  float* Cf = reinterpret_cast<float*>(C);
  const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(bias);
#define ELL_GEMM_CASE(BN_, AM_, BM_, OUT_, BIAS_)                                                             \
  if (BN == BN_ && (bool)a_mn == AM_ && (bool)b_mn == BM_ && out_mode == OUT_ && (bias != nullptr) == BIAS_) \
    return launch_gemm<BN_, AM_, BM_, OUT_, BIAS_>(tA, tB, tC, Cf, bp, M, N, K, ldc, err, ctas, stream);
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
