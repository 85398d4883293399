// Fused RMSNorm (optionally with the residual add of a pre-norm block) for sm_100a.
//
//   fwd :  h = x (+ residual);  y = h * rsqrt(mean(h^2) + eps) * w      (fp32 statistics)
//   bwd :  dh = rstd * (g - xhat * mean(g * xhat)) (+ dres),  g = dy * w,  xhat = h * rstd
//          dw = sum_rows dy * xhat   (per-CTA partials in scratch, then a column reduce)
//
// The op is HBM-bound: one read of each input and one write of each output per element.
// A warp owns one row at a time (hidden <= 8192), eight rows per CTA in flight;
// the grid is persistent and strides over rows.
// Replaces flash_attn.ops.rms_norm / dropout_layer_norm used by the reference
// (llm/models/mg_models/base_modules/layers/fused_layer_norm.py:49-57).
#include "common.cuh"

namespace ell {

// One warp per row (no block barriers on the critical path), two passes over the row: the second
// pass re-reads the 8-16 KB row from L1/L2.  8 rows are in flight per CTA, several CTAs per SM.
constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;
constexpr int kNormMaxCols = 8192;

template <bool kHasRes>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int rows, int cols,
                   float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = cols / 8;
  const bf16x8* wv = reinterpret_cast<const bf16x8*>(w);
  for (int r = blockIdx.x * kNormWarps + warp; r < rows; r += gridDim.x * kNormWarps) {
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)r * cols);
    const bf16x8* rr = kHasRes ? reinterpret_cast<const bf16x8*>(res + (size_t)r * cols) : nullptr;
    bf16x8* hr = kHasRes ? reinterpret_cast<bf16x8*>(h_out + (size_t)r * cols) : nullptr;
    float ss = 0.f;
#pragma unroll 4
    for (int c = lane; c < nvec; c += 32) {
      float v[8];
      unpack8(xr[c], v);
      if (kHasRes) {
        float t[8];
        unpack8(rr[c], t);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] += t[j];
        bf16x8 hp = pack8(v);      // the residual stream is stored in bf16: statistics use the rounded value
        hr[c] = hp;
        unpack8(hp, v);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)cols + eps);
    if (lane == 0) rstd_out[r] = rstd;
    const bf16x8* src = kHasRes ? hr : xr;
    bf16x8* yr = reinterpret_cast<bf16x8*>(y + (size_t)r * cols);
#pragma unroll 4
    for (int c = lane; c < nvec; c += 32) {
      float v[8], g[8], o[8];
      unpack8(src[c], v);
      unpack8(wv[c], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[j] * rstd * g[j];
      yr[c] = pack8(o);
    }
  }
}

// Backward: dw is accumulated per CTA in shared memory (fp32 atomics), then written as one partial row.
template <bool kHasDres>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dh,
                   float* __restrict__ dw_partial, int rows, int cols) {
  extern __shared__ float s_dw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = cols / 8;
  for (int c = threadIdx.x; c < cols; c += kNormThreads) s_dw[c] = 0.f;
  __syncthreads();
  const bf16x8* wv = reinterpret_cast<const bf16x8*>(w);
  for (int r = blockIdx.x * kNormWarps + warp; r < rows; r += gridDim.x * kNormWarps) {
    const float rstd = rstd_in[r];
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + (size_t)r * cols);
    const bf16x8* hr = reinterpret_cast<const bf16x8*>(h + (size_t)r * cols);
    float dot = 0.f;
#pragma unroll 2
    for (int c = lane; c < nvec; c += 32) {
      float d[8], x[8], g[8];
      unpack8(dyr[c], d);
      unpack8(hr[c], x);
      unpack8(wv[c], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = x[j] * rstd;
        dot += d[j] * g[j] * xh;
        atomicAdd(&s_dw[c * 8 + j], d[j] * xh);
      }
    }
    dot = warp_sum(dot) / (float)cols;
    bf16x8* dhr = reinterpret_cast<bf16x8*>(dh + (size_t)r * cols);
#pragma unroll 2
    for (int c = lane; c < nvec; c += 32) {
      float d[8], x[8], g[8], o[8];
      unpack8(dyr[c], d);
      unpack8(hr[c], x);
      unpack8(wv[c], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rstd * (d[j] * g[j] - x[j] * rstd * dot);
      if (kHasDres) {
        float t[8];
        unpack8(reinterpret_cast<const bf16x8*>(dres + (size_t)r * cols)[c], t);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += t[j];
      }
      dhr[c] = pack8(o);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += kNormThreads) dw_partial[(size_t)blockIdx.x * cols + c] = s_dw[c];
}

// dw[c] (+)= sum_p partial[p][c]; one thread per column, coalesced across the warp.
__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int parts,
                                         int cols, int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[(size_t)p * cols + c];
  dw[c] = accumulate ? dw[c] + s : s;
}

inline int norm_grid(int rows) {
  const int want = (rows + kNormWarps - 1) / kNormWarps;
  const int g = kNumSMs * 2;
  return want < g ? want : g;
}

}  // namespace ell

using namespace ell;

// Number of fp32 scratch elements rmsnorm_bwd needs for its per-CTA weight-gradient partials.
ELL_API long long ell_rmsnorm_bwd_scratch_elems(int rows, int cols) { return (long long)norm_grid(rows) * cols; }

ELL_API int ell_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                            int rows, int cols, float eps, cudaStream_t stream) {
  if (cols % 8 || cols > kNormMaxCols) return -1;
  if (rows == 0) return 0;
  dim3 grid((rows + kNormWarps - 1) / kNormWarps < kNumSMs * 8 ? (rows + kNormWarps - 1) / kNormWarps : kNumSMs * 8),
      block(kNormThreads);
  if (res)
    rmsnorm_fwd_kernel<true><<<grid, block, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res,
                                                         (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
                                                         (__nv_bfloat16*)h_out, rstd, rows, cols, eps);
  else
    rmsnorm_fwd_kernel<false><<<grid, block, 0, stream>>>((const __nv_bfloat16*)x, nullptr, (const __nv_bfloat16*)w,
                                                          (__nv_bfloat16*)y, nullptr, rstd, rows, cols, eps);
  return launch_status();
}

// dw is fp32 [cols]; `scratch` holds ell_rmsnorm_bwd_scratch_elems floats.
ELL_API int ell_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres,
                            void* dh, float* dw, float* scratch, int rows, int cols, int accumulate_dw,
                            cudaStream_t stream) {
  if (cols % 8 || cols > kNormMaxCols) return -1;
  if (rows == 0) return 0;
  const int parts = norm_grid(rows);
  dim3 grid(parts), block(kNormThreads);
  if (dres)
    rmsnorm_bwd_kernel<true><<<grid, block, cols * sizeof(float), stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)h,
                                                         (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
                                                         (__nv_bfloat16*)dh, scratch, rows, cols);
  else
    rmsnorm_bwd_kernel<false><<<grid, block, cols * sizeof(float), stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)h,
                                                          (const __nv_bfloat16*)w, rstd, nullptr, (__nv_bfloat16*)dh,
                                                          scratch, rows, cols);
  rmsnorm_dw_reduce_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(scratch, dw, parts, cols, accumulate_dw);
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the backward: the per-CTA partials live in a fixed device array.
// ---------------------------------------------------------------------------------------------
#include "no_alloc.h"

#include <mutex>

static __device__ __align__(256) float g_static_norm_scratch[ELL_STATIC_NORM_SCRATCH_ELEMS];

namespace {
constexpr int kStaticMaxDevices = 64;
float* g_static_scratch_ptr[kStaticMaxDevices] = {};
std::mutex g_static_mu;

// Device address of the scratch array on the current device; looked up once per device.
int static_scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) return ELL_STATIC_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_scratch_ptr[dev]) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_norm_scratch);
    if (e != cudaSuccess || !p) {
      (void)cudaGetLastError();
      return ELL_STATIC_ERR_SYMBOL;
    }
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return ELL_STATIC_OK;
}
}  // namespace

ELL_API const char* ell_static_strerror(int code) {
  switch (code) {
    case ELL_STATIC_OK: return "ok";
    case ELL_STATIC_ERR_SHAPE: return "rmsnorm_bwd_static: cols must be a positive multiple of 8 and rows >= 0";
    case ELL_STATIC_ERR_TOO_LARGE: return "rmsnorm_bwd_static: cols exceeds the fixed scratch (max 8192 columns)";
    case ELL_STATIC_ERR_SYMBOL: return "rmsnorm_bwd_static: cudaGetSymbolAddress failed for the scratch array";
    case ELL_STATIC_ERR_DEVICE: return "rmsnorm_bwd_static: no current CUDA device, or ordinal >= 64";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "rmsnorm_bwd_static: unknown error";
  }
}

ELL_API int ell_rmsnorm_bwd_static(const void* dy, const void* h, const void* w, const float* rstd, const void* dres,
                                   void* dh, float* dw, int rows, int cols, int accumulate_dw, cudaStream_t stream) {
  if (cols <= 0 || cols % 8 || rows < 0) return ELL_STATIC_ERR_SHAPE;
  if (cols > ELL_STATIC_NORM_MAX_COLS) return ELL_STATIC_ERR_TOO_LARGE;
  if (rows == 0) return ELL_STATIC_OK;
  float* scratch = nullptr;
  if (int rc = static_scratch_for_current_device(&scratch)) return rc;
  int parts = norm_grid(rows);
  const int cap = ELL_STATIC_NORM_SCRATCH_ELEMS / cols;   // >= 144 CTAs for every admitted cols
  if (parts > cap) parts = cap;
  dim3 grid(parts), block(kNormThreads);
  // Every partial row [0, parts) is written in full by the first kernel before the second reads it,
  // so stale contents of the shared scratch are never observed.
  if (dres)
    rmsnorm_bwd_kernel<true><<<grid, block, cols * sizeof(float), stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
        (__nv_bfloat16*)dh, scratch, rows, cols);
  else
    rmsnorm_bwd_kernel<false><<<grid, block, cols * sizeof(float), stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, rstd, nullptr, (__nv_bfloat16*)dh,
        scratch, rows, cols);
  rmsnorm_dw_reduce_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(scratch, dw, parts, cols, accumulate_dw);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? ELL_STATIC_OK : (int)e;
}
