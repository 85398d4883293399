// Affine LayerNorm (optionally with the residual add of a pre-norm block) for sm_100a, mixed precision:
// bf16 activations and parameters, fp32 statistics and parameter gradients.
//
//   fwd :  h = x (+ residual);  y = (h - mean(h)) * rsqrt(var(h) + eps) * w + b
//   bwd :  g = dy * w,  xhat = (h - mean) * rstd
//          dh = rstd * (g - mean(g) - xhat * mean(g * xhat)) (+ dres)
//          dw += sum_rows dy * xhat,  db += sum_rows dy          (fp32, accumulated into the caller's buffers)
//
// A warp owns one row: it reads the row once for the statistics and a second time (from L1 / L2) to normalise, so
// any hidden size that is a multiple of 8 works without a register budget per column.  The parameter gradients are
// a separate column-sum pass over dy and h (blocks of 256 columns x row slices, one fp32 atomic per column and block).
// The Llama presets use RMSNorm (norm.cu); this kernel serves `layer_norm_params.type: layer_norm`.
// Replaces fused_mix_prec_layer_norm_cuda.forward_affine / backward_affine of the reference
// (llm/models/mg_models/base_modules/layers/fused_layer_norm.py:74-140).
#include "common.cuh"

namespace ell {

constexpr int kLnThreads = 256;
constexpr int kLnWarps = kLnThreads / 32;

template <bool kHasRes>
__global__ void __launch_bounds__(kLnThreads)
layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                     const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                     __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out, float* __restrict__ mean_out,
                     float* __restrict__ rstd_out, int rows, int cols, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = cols / 8;
  for (int r = blockIdx.x * kLnWarps + warp; r < rows; r += gridDim.x * kLnWarps) {
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)r * cols);
    const bf16x8* rr = kHasRes ? reinterpret_cast<const bf16x8*>(res + (size_t)r * cols) : nullptr;
    bf16x8* hr = kHasRes ? reinterpret_cast<bf16x8*>(h_out + (size_t)r * cols) : nullptr;
    float s = 0.f;
    for (int c = lane; c < nvec; c += 32) {
      float v[8];
      unpack8(xr[c], v);
      if (kHasRes) {
        float t[8];
        unpack8(rr[c], t);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] += t[j];
        const bf16x8 hv = pack8(v);          // the residual stream is stored in bf16: statistics use the rounded value
        hr[c] = hv;
        unpack8(hv, v);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[j];
    }
    const float mean = warp_sum(s) / (float)cols;
    const bf16x8* src = kHasRes ? reinterpret_cast<const bf16x8*>(hr) : xr;
    __syncwarp();                            // this warp's h_out stores are visible to its own re-read
    float q = 0.f;
    for (int c = lane; c < nvec; c += 32) {
      float v[8];
      unpack8(src[c], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) q += (v[j] - mean) * (v[j] - mean);
    }
    const float rstd = rsqrtf(warp_sum(q) / (float)cols + eps);
    if (lane == 0) {
      mean_out[r] = mean;
      rstd_out[r] = rstd;
    }
    bf16x8* yr = reinterpret_cast<bf16x8*>(y + (size_t)r * cols);
    for (int c = lane; c < nvec; c += 32) {
      float v[8], g[8], bb[8], o[8];
      unpack8(src[c], v);
      unpack8(reinterpret_cast<const bf16x8*>(w)[c], g);
      unpack8(reinterpret_cast<const bf16x8*>(b)[c], bb);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[j] - mean) * rstd * g[j] + bb[j];
      yr[c] = pack8(o);
    }
  }
}

template <bool kHasDres>
__global__ void __launch_bounds__(kLnThreads)
layernorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean,
                        const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dres,
                        __nv_bfloat16* __restrict__ dh, int rows, int cols) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = cols / 8;
  for (int r = blockIdx.x * kLnWarps + warp; r < rows; r += gridDim.x * kLnWarps) {
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + (size_t)r * cols);
    const bf16x8* hr = reinterpret_cast<const bf16x8*>(h + (size_t)r * cols);
    const float mu = mean[r], rs = rstd[r];
    float sg = 0.f, sgx = 0.f;
    for (int c = lane; c < nvec; c += 32) {
      float d[8], v[8], g[8];
      unpack8(dyr[c], d);
      unpack8(hr[c], v);
      unpack8(reinterpret_cast<const bf16x8*>(w)[c], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gj = d[j] * g[j];
        sg += gj;
        sgx += gj * (v[j] - mu) * rs;
      }
    }
    const float mg = warp_sum(sg) / (float)cols, mgx = warp_sum(sgx) / (float)cols;
    bf16x8* dhr = reinterpret_cast<bf16x8*>(dh + (size_t)r * cols);
    const bf16x8* drr = kHasDres ? reinterpret_cast<const bf16x8*>(dres + (size_t)r * cols) : nullptr;
    for (int c = lane; c < nvec; c += 32) {
      float d[8], v[8], g[8], o[8];
      unpack8(dyr[c], d);
      unpack8(hr[c], v);
      unpack8(reinterpret_cast<const bf16x8*>(w)[c], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (d[j] * g[j] - mg - (v[j] - mu) * rs * mgx);
      if (kHasDres) {
        float t[8];
        unpack8(drr[c], t);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += t[j];
      }
      dhr[c] = pack8(o);
    }
  }
}

// dw[c] += sum_r dy[r,c] * (h[r,c] - mean[r]) * rstd[r];  db[c] += sum_r dy[r,c]
__global__ void __launch_bounds__(256)
layernorm_bwd_dwdb_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                          const float* __restrict__ mean, const float* __restrict__ rstd, float* __restrict__ dw,
                          float* __restrict__ db, int rows, int cols) {
  __shared__ float red_w[8][256], red_b[8][256];
  const int cg = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 256 + cg * 8;
  float aw[8], ab[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) aw[e] = ab[e] = 0.f;
  if (c0 < cols) {
    for (int r = blockIdx.y * 8 + rl; r < rows; r += gridDim.y * 8) {
      float d[8], v[8];
      unpack8(*reinterpret_cast<const bf16x8*>(dy + (size_t)r * cols + c0), d);
      unpack8(*reinterpret_cast<const bf16x8*>(h + (size_t)r * cols + c0), v);
      const float mu = mean[r], rs = rstd[r];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        aw[e] += d[e] * (v[e] - mu) * rs;
        ab[e] += d[e];
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    red_w[rl][cg * 8 + e] = aw[e];
    red_b[rl][cg * 8 + e] = ab[e];
  }
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < cols) {
    float sw = 0.f, sb = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sw += red_w[i][threadIdx.x];
      sb += red_b[i][threadIdx.x];
    }
    atomicAdd(dw + c, sw);
    atomicAdd(db + c, sb);
  }
}

static int ln_grid(int rows) {
  const int need = (rows + kLnWarps - 1) / kLnWarps;
  return need < kNumSMs * 8 ? need : kNumSMs * 8;
}

}  // namespace ell

using namespace ell;

// y = LayerNorm(x (+ residual)) * w + b.  h_out (the sum, bf16) is written only with a residual.  mean / rstd: fp32
// [rows], kept for the backward.  cols must be a multiple of 8.
ELL_API int ell_layernorm_fwd(const void* x, const void* residual, const void* w, const void* b, void* y, void* h_out,
                              float* mean, float* rstd, int rows, int cols, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (cols <= 0 || cols % 8) return -1;
  if (residual)
    layernorm_fwd_kernel<true><<<ln_grid(rows), kLnThreads, 0, stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b,
        (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, mean, rstd, rows, cols, eps);
  else
    layernorm_fwd_kernel<false><<<ln_grid(rows), kLnThreads, 0, stream>>>(
        (const __nv_bfloat16*)x, nullptr, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, nullptr,
        mean, rstd, rows, cols, eps);
  return launch_status();
}

// dh = d(loss)/dh (+ dres); dw32 / db32 [cols] fp32 are ACCUMULATED into (zero them, or pass the fp32 main_grad).
ELL_API int ell_layernorm_bwd(const void* dy, const void* h, const void* w, const float* mean, const float* rstd,
                              const void* dres, void* dh, float* dw32, float* db32, int rows, int cols,
                              cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (cols <= 0 || cols % 8) return -1;
  if (dres)
    layernorm_bwd_dx_kernel<true><<<ln_grid(rows), kLnThreads, 0, stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, mean, rstd,
        (const __nv_bfloat16*)dres, (__nv_bfloat16*)dh, rows, cols);
  else
    layernorm_bwd_dx_kernel<false><<<ln_grid(rows), kLnThreads, 0, stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, mean, rstd, nullptr,
        (__nv_bfloat16*)dh, rows, cols);
  int rc = launch_status();
  if (rc) return rc;
  const int bx = (cols + 255) / 256;
  int by = (rows + 63) / 64;
  const int cap = (kNumSMs * 8 + bx - 1) / bx;
  if (by > cap) by = cap;
  if (by < 1) by = 1;
  layernorm_bwd_dwdb_kernel<<<dim3(bx, by), 256, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, mean,
                                                              rstd, dw32, db32, rows, cols);
  return launch_status();
}
