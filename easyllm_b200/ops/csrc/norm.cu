// Fused RMSNorm (optionally with the residual add of a pre-norm block) for sm_100a.
//
//   fwd :  h = x (+ residual);  y = h * rsqrt(mean(h^2) + eps) * w      (fp32 statistics)
//   bwd :  dh = rstd * (g - xhat * mean(g * xhat)) (+ dres),  g = dy * w,  xhat = h * rstd
//          dw = sum_rows dy * xhat   (per-CTA partials in scratch, then a column reduce)
//
// The op is HBM-bound: one read of each input and one write of each output per element.
// A CTA of 256 threads owns one row at a time and keeps it in registers (hidden <= 8192);
// the grid is persistent (a multiple of the SM count) and strides over rows.
// Replaces flash_attn.ops.rms_norm / dropout_layer_norm used by the reference
// (llm/models/mg_models/base_modules/layers/fused_layer_norm.py:49-57).
#include "common.cuh"

namespace ell {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // 256 threads * 4 * 8 elements = 8192 columns

template <bool kHasRes>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int rows, int cols,
                   float eps) {
  __shared__ float red[33];
  const int nvec = cols / 8;
  float wv[kNormMaxVec][8];
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    int c = threadIdx.x + i * kNormThreads;
    if (c < nvec) unpack8(reinterpret_cast<const bf16x8*>(w)[c], wv[i]);
  }
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)r * cols);
    const bf16x8* rr = kHasRes ? reinterpret_cast<const bf16x8*>(res + (size_t)r * cols) : nullptr;
    float v[kNormMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      int c = threadIdx.x + i * kNormThreads;
      if (c < nvec) {
        unpack8(xr[c], v[i]);
        if (kHasRes) {
          float t[8];
          unpack8(rr[c], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += t[j];
          // the residual stream is stored in bf16: statistics use the rounded value
          bf16x8 hp = pack8(v[i]);
          reinterpret_cast<bf16x8*>(h_out + (size_t)r * cols)[c] = hp;
          unpack8(hp, v[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)cols + eps);
    if (threadIdx.x == 0) rstd_out[r] = rstd;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      int c = threadIdx.x + i * kNormThreads;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[i][j];
        reinterpret_cast<bf16x8*>(y + (size_t)r * cols)[c] = pack8(o);
      }
    }
  }
}

template <bool kHasDres>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dh,
                   float* __restrict__ dw_partial, int rows, int cols) {
  __shared__ float red[33];
  const int nvec = cols / 8;
  float wv[kNormMaxVec][8], dwacc[kNormMaxVec][8];
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    int c = threadIdx.x + i * kNormThreads;
    if (c < nvec) unpack8(reinterpret_cast<const bf16x8*>(w)[c], wv[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  }
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float rstd = rstd_in[r];
    float g[kNormMaxVec][8], xh[kNormMaxVec][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      int c = threadIdx.x + i * kNormThreads;
      if (c < nvec) {
        float d[8];
        unpack8(reinterpret_cast<const bf16x8*>(dy + (size_t)r * cols)[c], d);
        unpack8(reinterpret_cast<const bf16x8*>(h + (size_t)r * cols)[c], xh[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rstd;
          dwacc[i][j] += d[j] * xh[i][j];
          g[i][j] = d[j] * wv[i][j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    dot = block_sum(dot, red) / (float)cols;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      int c = threadIdx.x + i * kNormThreads;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * dot);
        if (kHasDres) {
          float t[8];
          unpack8(reinterpret_cast<const bf16x8*>(dres + (size_t)r * cols)[c], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += t[j];
        }
        reinterpret_cast<bf16x8*>(dh + (size_t)r * cols)[c] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    int c = threadIdx.x + i * kNormThreads;
    if (c < nvec) {
      float4* dst = reinterpret_cast<float4*>(dw_partial + (size_t)blockIdx.x * cols + (size_t)c * 8);
      dst[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      dst[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
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
  int g = kNumSMs * 4;
  return rows < g ? rows : g;
}

}  // namespace ell

using namespace ell;

// Number of fp32 scratch elements rmsnorm_bwd needs for its per-CTA weight-gradient partials.
ELL_API long long ell_rmsnorm_bwd_scratch_elems(int rows, int cols) { return (long long)norm_grid(rows) * cols; }

ELL_API int ell_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                            int rows, int cols, float eps, cudaStream_t stream) {
  if (cols % 8 || cols > kNormThreads * kNormMaxVec * 8) return -1;
  if (rows == 0) return 0;
  dim3 grid(norm_grid(rows)), block(kNormThreads);
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
  if (cols % 8 || cols > kNormThreads * kNormMaxVec * 8) return -1;
  if (rows == 0) return 0;
  const int parts = norm_grid(rows);
  dim3 grid(parts), block(kNormThreads);
  if (dres)
    rmsnorm_bwd_kernel<true><<<grid, block, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)h,
                                                         (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
                                                         (__nv_bfloat16*)dh, scratch, rows, cols);
  else
    rmsnorm_bwd_kernel<false><<<grid, block, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)h,
                                                          (const __nv_bfloat16*)w, rstd, nullptr, (__nv_bfloat16*)dh,
                                                          scratch, rows, cols);
  rmsnorm_dw_reduce_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(scratch, dw, parts, cols, accumulate_dw);
  return launch_status();
}
