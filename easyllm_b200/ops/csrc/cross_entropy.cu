// Vocab-parallel softmax cross-entropy over bf16 logits, for sm_100a.
//
//   fwd  : per token, one online-softmax pass over this rank's vocab shard gives
//          (row max, sum exp(l - max), target logit or 0) -> parts[T][3] (fp32).
//          The three scalars per token are what is combined across tensor-parallel ranks
//          (max, then rescaled sums) instead of three all-reduces over full rows.
//   bwd  : dlogits = (exp(l - lse) - onehot(target)) * scale[token], written in place over the
//          logits (bf16), lse being the global log-sum-exp.
//
// The reference casts logits to fp32 and runs ~12 eager kernels plus 3 all-reduces
// (llm/models/mg_models/base_modules/functions/cross_entropy.py:22-112); here logits stay
// bf16 in HBM and every element is read once per pass.
#include "common.cuh"

namespace ell {

constexpr int kCeThreads = 256;

__global__ void __launch_bounds__(kCeThreads)
ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
              float* __restrict__ parts, int T, int ld, int valid_cols, long long vocab_start) {
  __shared__ float red[33];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const __nv_bfloat16* row = logits + (size_t)t * ld;
    float mx = -INFINITY, se = 0.f;
    const int nv = valid_cols / 8;
    for (int c = threadIdx.x; c < nv; c += kCeThreads) {
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(row)[c], f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      if (lm > mx) {
        se *= __expf(mx - lm);
        mx = lm;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) se += __expf(f[j] - mx);
    }
    for (int c = nv * 8 + threadIdx.x; c < valid_cols; c += kCeThreads) {
      float f = __bfloat162float(row[c]);
      if (f > mx) {
        se *= __expf(mx - f);
        mx = f;
      }
      se += __expf(f - mx);
    }
    const float gmx = block_max(mx, red);
    se = (mx == -INFINITY) ? 0.f : se * __expf(mx - gmx);
    se = block_sum(se, red);
    if (threadIdx.x == 0) {
      const long long loc = target[t] - vocab_start;
      float tl = 0.f;
      if (loc >= 0 && loc < valid_cols) tl = __bfloat162float(row[loc]);
      parts[(size_t)t * 3 + 0] = gmx;
      parts[(size_t)t * 3 + 1] = se;
      parts[(size_t)t * 3 + 2] = tl;
    }
  }
}

// Columns >= valid_cols (padded vocab tail) receive zero gradient.
__global__ void __launch_bounds__(kCeThreads)
ce_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
              const float* __restrict__ lse, const float* __restrict__ scale, int T, int ld, int cols,
              int valid_cols, long long vocab_start) {
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __nv_bfloat16* row = logits + (size_t)t * ld;
    const float l = lse[t], s = scale[t];
    const long long loc = target[t] - vocab_start;
    const int nv = cols / 8;
    for (int c = threadIdx.x; c < nv; c += kCeThreads) {
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(row)[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = c * 8 + j;
        float p = col < valid_cols ? __expf(f[j] - l) : 0.f;
        if (col == loc) p -= 1.f;
        f[j] = p * s;
      }
      reinterpret_cast<bf16x8*>(row)[c] = pack8(f);
    }
    for (int col = nv * 8 + threadIdx.x; col < cols; col += kCeThreads) {
      float p = col < valid_cols ? __expf(__bfloat162float(row[col]) - l) : 0.f;
      if (col == loc) p -= 1.f;
      row[col] = __float2bfloat16_rn(p * s);
    }
  }
}

}  // namespace ell

using namespace ell;

ELL_API int ell_ce_fwd(const void* logits, const long long* target, float* parts, int T, int ld, int valid_cols,
                       long long vocab_start, cudaStream_t stream) {
  if (T == 0) return 0;
  if (ld % 8) return -1;
  int grid = T < kNumSMs * 8 ? T : kNumSMs * 8;
  ce_fwd_kernel<<<grid, kCeThreads, 0, stream>>>((const __nv_bfloat16*)logits, target, parts, T, ld, valid_cols,
                                                 vocab_start);
  return launch_status();
}

ELL_API int ell_ce_bwd(void* logits, const long long* target, const float* lse, const float* scale, int T, int ld,
                       int cols, int valid_cols, long long vocab_start, cudaStream_t stream) {
  if (T == 0) return 0;
  if (ld % 8) return -1;
  int grid = T < kNumSMs * 8 ? T : kNumSMs * 8;
  ce_bwd_kernel<<<grid, kCeThreads, 0, stream>>>((__nv_bfloat16*)logits, target, lse, scale, T, ld, cols, valid_cols,
                                                 vocab_start);
  return launch_status();
}

namespace ell {
// parts[T, 3] = merge over column tiles of part[tiles][3][T] (max, sum-exp relative to that max, target logit).
__global__ void ce_combine_kernel(const float* __restrict__ part, float* __restrict__ parts, int tiles, int T) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float m = -INFINITY, s = 0.f, tl = 0.f;
  for (int i = 0; i < tiles; ++i) {
    const float* p = part + (size_t)i * 3 * T + t;
    const float mi = p[0], si = p[(size_t)T];
    tl += p[(size_t)2 * T];
    if (mi > -INFINITY) {
      const float nm = fmaxf(m, mi);
      s = s * __expf(m - nm) + si * __expf(mi - nm);
      m = nm;
    }
  }
  parts[(size_t)t * 3] = m;
  parts[(size_t)t * 3 + 1] = s;
  parts[(size_t)t * 3 + 2] = tl;
}
}  // namespace ell

ELL_API int ell_ce_combine(const float* part, float* parts, int tiles, int T, cudaStream_t stream) {
  if (T == 0) return 0;
  ell::ce_combine_kernel<<<(T + 255) / 256, 256, 0, stream>>>(part, parts, tiles, T);
  return ell::launch_status();
}
