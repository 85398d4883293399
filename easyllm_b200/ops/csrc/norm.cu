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

// A CTA of 256 threads owns kNormRows rows at a time; thread t holds the 16-byte vectors t, t+256, ... of
// each row in registers (kVpt <= 4 vectors for hidden <= 8192), so every element is read from HBM exactly
// once and never re-read from L1/L2.  The next rows are prefetched into registers before the current ones
// are reduced, which keeps ~64 KB per SM in flight across the one block barrier per iteration.
constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;
constexpr int kNormMaxCols = 8192;
// Rows per CTA iteration and CTAs per SM by vectors per thread: the register file bounds what can be in flight.
__host__ __device__ constexpr int norm_rows(int vpt) { return vpt <= 2 ? 2 : 1; }
__host__ __device__ constexpr int norm_min_ctas(int vpt) { return vpt <= 1 ? 3 : 2; }
constexpr int kNormRowsMax = 2;

__host__ __device__ constexpr int norm_rows_bwd(int vpt) { return vpt <= 1 ? 2 : 1; }
__host__ __device__ constexpr int norm_min_ctas_bwd(int vpt) { return vpt <= 2 ? 2 : 1; }

template <int kVpt, int kNormRows>
struct RowRegs {
  bf16x8 v[kNormRows][kVpt];
};

template <int kVpt, int kNormRows>
__device__ __forceinline__ void load_rows(RowRegs<kVpt, kNormRows>& d, const __nv_bfloat16* __restrict__ base, int r0, int rows,
                                          int cols, int nvec) {
#pragma unroll
  for (int k = 0; k < kNormRows; ++k)
#pragma unroll
    for (int i = 0; i < kVpt; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      if (r0 + k < rows && c < nvec)
        d.v[k][i] = reinterpret_cast<const bf16x8*>(base + (size_t)(r0 + k) * cols)[c];
      else
        d.v[k][i] = bf16x8{};
    }
}

// Sum over the CTA of kNormRows partials; `red` is one of two alternating buffers (one barrier per call).
template <int kNormRows>
__device__ __forceinline__ void rows_block_sum(float (&p)[kNormRows], float (*red)[kNormRowsMax]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int k = 0; k < kNormRows; ++k) {
    p[k] = warp_sum(p[k]);
    if (lane == 0) red[warp][k] = p[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kNormRows; ++k) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kNormWarps; ++w) t += red[w][k];
    p[k] = t;
  }
}

template <int kVpt, bool kHasRes>
__global__ void __launch_bounds__(kNormThreads, norm_min_ctas(kVpt))
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int rows, int cols,
                   float eps) {
  __shared__ float s_red[2][kNormWarps][kNormRowsMax];
  constexpr int kNormRows = norm_rows(kVpt);
  const int nvec = cols / 8;
  bf16x8 wv[kVpt];
#pragma unroll
  for (int i = 0; i < kVpt; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    wv[i] = c < nvec ? reinterpret_cast<const bf16x8*>(w)[c] : bf16x8{};
  }
  const int stride = gridDim.x * kNormRows;
  int r0 = blockIdx.x * kNormRows;
  RowRegs<kVpt, kNormRows> nx, nr;
  load_rows<kVpt, kNormRows>(nx, x, r0, rows, cols, nvec);
  if (kHasRes) load_rows<kVpt, kNormRows>(nr, res, r0, rows, cols, nvec);
  for (int it = 0; r0 < rows; r0 += stride, ++it) {
    RowRegs<kVpt, kNormRows> cx = nx, cr;
    if (kHasRes) cr = nr;
    load_rows<kVpt, kNormRows>(nx, x, r0 + stride, rows, cols, nvec);
    if (kHasRes) load_rows<kVpt, kNormRows>(nr, res, r0 + stride, rows, cols, nvec);
    float ss[kNormRows];
#pragma unroll
    for (int k = 0; k < kNormRows; ++k) {
      ss[k] = 0.f;
#pragma unroll
      for (int i = 0; i < kVpt; ++i) {
        const int c = threadIdx.x + i * kNormThreads;
        float v[8];
        unpack8(cx.v[k][i], v);
        if (kHasRes) {
          float t[8];
          unpack8(cr.v[k][i], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += t[j];
          cx.v[k][i] = pack8(v);   // the residual stream is stored in bf16: statistics use the rounded value
          if (r0 + k < rows && c < nvec) reinterpret_cast<bf16x8*>(h_out + (size_t)(r0 + k) * cols)[c] = cx.v[k][i];
          unpack8(cx.v[k][i], v);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss[k] += v[j] * v[j];
      }
    }
    rows_block_sum<kNormRows>(ss, s_red[it & 1]);
#pragma unroll
    for (int k = 0; k < kNormRows; ++k) {
      if (r0 + k >= rows) break;
      const float rstd = rsqrtf(ss[k] / (float)cols + eps);
      if (threadIdx.x == 0) rstd_out[r0 + k] = rstd;
#pragma unroll
      for (int i = 0; i < kVpt; ++i) {
        const int c = threadIdx.x + i * kNormThreads;
        if (c >= nvec) break;
        float v[8], g[8], o[8];
        unpack8(cx.v[k][i], v);
        unpack8(wv[i], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[j] * rstd * g[j];
        reinterpret_cast<bf16x8*>(y + (size_t)(r0 + k) * cols)[c] = pack8(o);
      }
    }
  }
}

// Backward: each thread accumulates dw for the columns it owns in registers over all rows of the CTA and
// writes them once as this CTA's partial row.
template <int kVpt, bool kHasDres>
__global__ void __launch_bounds__(kNormThreads, norm_min_ctas_bwd(kVpt))
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dh,
                   float* __restrict__ dw_partial, int rows, int cols) {
  __shared__ float s_red[2][kNormWarps][kNormRowsMax];
  constexpr int kNormRows = norm_rows_bwd(kVpt);
  const int nvec = cols / 8;
  bf16x8 wv[kVpt];
  float dw[kVpt][8];
#pragma unroll
  for (int i = 0; i < kVpt; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    wv[i] = c < nvec ? reinterpret_cast<const bf16x8*>(w)[c] : bf16x8{};
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[i][j] = 0.f;
  }
  const int stride = gridDim.x * kNormRows;
  int r0 = blockIdx.x * kNormRows;
  RowRegs<kVpt, kNormRows> nd, nh;
  load_rows<kVpt, kNormRows>(nd, dy, r0, rows, cols, nvec);
  load_rows<kVpt, kNormRows>(nh, h, r0, rows, cols, nvec);
  for (int it = 0; r0 < rows; r0 += stride, ++it) {
    RowRegs<kVpt, kNormRows> cd = nd, ch = nh, cres;
    float rstd[kNormRows];
#pragma unroll
    for (int k = 0; k < kNormRows; ++k) rstd[k] = r0 + k < rows ? rstd_in[r0 + k] : 0.f;
    if (kHasDres) load_rows<kVpt, kNormRows>(cres, dres, r0, rows, cols, nvec);
    load_rows<kVpt, kNormRows>(nd, dy, r0 + stride, rows, cols, nvec);
    load_rows<kVpt, kNormRows>(nh, h, r0 + stride, rows, cols, nvec);
    float dot[kNormRows];
#pragma unroll
    for (int k = 0; k < kNormRows; ++k) {
      dot[k] = 0.f;
#pragma unroll
      for (int i = 0; i < kVpt; ++i) {
        float d[8], x[8], g[8];
        unpack8(cd.v[k][i], d);
        unpack8(ch.v[k][i], x);
        unpack8(wv[i], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = x[j] * rstd[k];
          dot[k] += d[j] * g[j] * xh;
          dw[i][j] += d[j] * xh;
        }
      }
    }
    rows_block_sum<kNormRows>(dot, s_red[it & 1]);
#pragma unroll
    for (int k = 0; k < kNormRows; ++k) {
      if (r0 + k >= rows) break;
      const float m = dot[k] / (float)cols;
#pragma unroll
      for (int i = 0; i < kVpt; ++i) {
        const int c = threadIdx.x + i * kNormThreads;
        if (c >= nvec) break;
        float d[8], x[8], g[8], o[8];
        unpack8(cd.v[k][i], d);
        unpack8(ch.v[k][i], x);
        unpack8(wv[i], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd[k] * (d[j] * g[j] - x[j] * rstd[k] * m);
        if (kHasDres) {
          float t[8];
          unpack8(cres.v[k][i], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += t[j];
        }
        reinterpret_cast<bf16x8*>(dh + (size_t)(r0 + k) * cols)[c] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kVpt; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    if (c >= nvec) break;
    float4* dst = reinterpret_cast<float4*>(dw_partial + (size_t)blockIdx.x * cols + (size_t)c * 8);
    dst[0] = make_float4(dw[i][0], dw[i][1], dw[i][2], dw[i][3]);
    dst[1] = make_float4(dw[i][4], dw[i][5], dw[i][6], dw[i][7]);
  }
}

// dw[c] (+)= sum_p partial[p][c].  A block covers 32 columns with 8 warps; warp y sums the partial rows y, y + 8, ...
// (128 contiguous bytes per row and warp), the eight sums meet in shared memory in a fixed order.  128 blocks for
// 4096 columns instead of one thread per column walking all rows alone.
constexpr int kDwReduceCols = 32, kDwReduceWarps = 8;
__global__ void __launch_bounds__(kDwReduceCols * kDwReduceWarps)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int parts, int cols,
                         int accumulate) {
  __shared__ float red[kDwReduceWarps][kDwReduceCols];
  const int cx = threadIdx.x & 31, py = threadIdx.x >> 5;
  const int c = blockIdx.x * kDwReduceCols + cx;
  float s0 = 0.f, s1 = 0.f;
  if (c < cols) {
    int p = py;
    for (; p + kDwReduceWarps < parts; p += 2 * kDwReduceWarps) {
      s0 += partial[(size_t)p * cols + c];
      s1 += partial[(size_t)(p + kDwReduceWarps) * cols + c];
    }
    if (p < parts) s0 += partial[(size_t)p * cols + c];
  }
  red[py][cx] = s0 + s1;
  __syncthreads();
  if (py == 0 && c < cols) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kDwReduceWarps; ++i) s += red[i][cx];
    dw[c] = accumulate ? dw[c] + s : s;
  }
}

// Persistent grid for the backward: a few CTAs per SM, never more than there are row groups.
inline int norm_vpt(int cols) { return (cols / 8 + kNormThreads - 1) / kNormThreads; }

inline int norm_grid(int rows, int cols, bool bwd) {
  const int v = norm_vpt(cols);
  const int r = bwd ? norm_rows_bwd(v) : norm_rows(v);
  const int want = (rows + r - 1) / r;
  const int g = kNumSMs * (bwd ? norm_min_ctas_bwd(v) : norm_min_ctas(v));
  return want < g ? want : g;
}

template <bool kHasRes>
void launch_norm_fwd(int vpt, dim3 grid, cudaStream_t stream, const __nv_bfloat16* x, const __nv_bfloat16* res,
                     const __nv_bfloat16* w, __nv_bfloat16* y, __nv_bfloat16* h_out, float* rstd, int rows, int cols,
                     float eps) {
  dim3 block(kNormThreads);
  switch (vpt) {
    case 1: rmsnorm_fwd_kernel<1, kHasRes><<<grid, block, 0, stream>>>(x, res, w, y, h_out, rstd, rows, cols, eps); break;
    case 2: rmsnorm_fwd_kernel<2, kHasRes><<<grid, block, 0, stream>>>(x, res, w, y, h_out, rstd, rows, cols, eps); break;
    case 3: rmsnorm_fwd_kernel<3, kHasRes><<<grid, block, 0, stream>>>(x, res, w, y, h_out, rstd, rows, cols, eps); break;
    default: rmsnorm_fwd_kernel<4, kHasRes><<<grid, block, 0, stream>>>(x, res, w, y, h_out, rstd, rows, cols, eps); break;
  }
}

template <bool kHasDres>
void launch_norm_bwd(int vpt, dim3 grid, cudaStream_t stream, const __nv_bfloat16* dy, const __nv_bfloat16* h,
                     const __nv_bfloat16* w, const float* rstd, const __nv_bfloat16* dres, __nv_bfloat16* dh,
                     float* partial, int rows, int cols) {
  dim3 block(kNormThreads);
  switch (vpt) {
    case 1: rmsnorm_bwd_kernel<1, kHasDres><<<grid, block, 0, stream>>>(dy, h, w, rstd, dres, dh, partial, rows, cols); break;
    case 2: rmsnorm_bwd_kernel<2, kHasDres><<<grid, block, 0, stream>>>(dy, h, w, rstd, dres, dh, partial, rows, cols); break;
    case 3: rmsnorm_bwd_kernel<3, kHasDres><<<grid, block, 0, stream>>>(dy, h, w, rstd, dres, dh, partial, rows, cols); break;
    default: rmsnorm_bwd_kernel<4, kHasDres><<<grid, block, 0, stream>>>(dy, h, w, rstd, dres, dh, partial, rows, cols); break;
  }
}

// Both kernels and the column reduce for `parts` CTAs; `partial` holds parts * cols floats.
inline void run_norm_bwd(int parts, cudaStream_t stream, const void* dy, const void* h, const void* w, const float* rstd,
                         const void* dres, void* dh, float* dw, float* partial, int rows, int cols, int accumulate_dw) {
  if (dres)
    launch_norm_bwd<true>(norm_vpt(cols), dim3(parts), stream, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h,
                          (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dh, partial, rows, cols);
  else
    launch_norm_bwd<false>(norm_vpt(cols), dim3(parts), stream, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h,
                           (const __nv_bfloat16*)w, rstd, nullptr, (__nv_bfloat16*)dh, partial, rows, cols);
  rmsnorm_dw_reduce_kernel<<<(cols + kDwReduceCols - 1) / kDwReduceCols, kDwReduceCols * kDwReduceWarps, 0, stream>>>(
      partial, dw, parts, cols, accumulate_dw);
}

}  // namespace ell

using namespace ell;

// Number of fp32 scratch elements rmsnorm_bwd needs for its per-CTA weight-gradient partials.
ELL_API long long ell_rmsnorm_bwd_scratch_elems(int rows, int cols) { return (long long)norm_grid(rows, cols, true) * cols; }

ELL_API int ell_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                            int rows, int cols, float eps, cudaStream_t stream) {
  if (cols % 8 || cols > kNormMaxCols) return -1;
  if (rows == 0) return 0;
  dim3 grid(norm_grid(rows, cols, false));
  if (res)
    launch_norm_fwd<true>(norm_vpt(cols), grid, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)res,
                          (const __nv_bfloat16*)w, (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, rstd, rows, cols, eps);
  else
    launch_norm_fwd<false>(norm_vpt(cols), grid, stream, (const __nv_bfloat16*)x, nullptr, (const __nv_bfloat16*)w,
                           (__nv_bfloat16*)y, nullptr, rstd, rows, cols, eps);
  return launch_status();
}

// dw is fp32 [cols]; `scratch` holds ell_rmsnorm_bwd_scratch_elems floats.
ELL_API int ell_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres,
                            void* dh, float* dw, float* scratch, int rows, int cols, int accumulate_dw,
                            cudaStream_t stream) {
  if (cols % 8 || cols > kNormMaxCols) return -1;
  if (rows == 0) {
    if (!accumulate_dw && dw) cudaMemsetAsync(dw, 0, sizeof(float) * (size_t)cols, stream);
    return launch_status();
  }
  run_norm_bwd(norm_grid(rows, cols, true), stream, dy, h, w, rstd, dres, dh, dw, scratch, rows, cols, accumulate_dw);
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
  if (rows == 0) {
    // no rows: the sum over rows is empty, so a dw that is not accumulated into becomes zero (a memset allocates nothing)
    if (!accumulate_dw && dw) {
      cudaError_t e = cudaMemsetAsync(dw, 0, sizeof(float) * (size_t)cols, stream);
      if (e != cudaSuccess) return (int)e;
    }
    return ELL_STATIC_OK;
  }
  float* scratch = nullptr;
  if (int rc = static_scratch_for_current_device(&scratch)) return rc;
  int parts = norm_grid(rows, cols, true);
  const int cap = ELL_STATIC_NORM_SCRATCH_ELEMS / cols;   // >= 144 CTAs for every admitted cols
  if (parts > cap) parts = cap;
  // Every partial row [0, parts) is written in full by the first kernel before the second reads it,
  // so stale contents of the shared scratch are never observed.
  run_norm_bwd(parts, stream, dy, h, w, rstd, dres, dh, dw, scratch, rows, cols, accumulate_dw);
  return launch_status();                                 // 0 == ELL_STATIC_OK, else the cudaError_t of the launch
}
