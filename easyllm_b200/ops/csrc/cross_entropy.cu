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

#include "gemm_fuse.cuh"

namespace ell {
constexpr int kCeTpThreads = 256;
constexpr int kErrCeExchange = 21;

// Cross-rank combine of the vocab-parallel cross-entropy statistics in one kernel, over peer memory.
// Every rank holds parts[T][3] = (max, sum exp(x - max), target logit) of its vocabulary shard.  A CTA pushes the
// triples of its 256 tokens into slot [parity][rank] of every peer's exchange buffer (plain stores over NVLink),
// raises a per-(source, CTA) epoch flag on the peer, waits (bounded) for the peers' flags of the same token block
// and merges the tp triples in rank order: out[0][t] = log-sum-exp over the whole vocabulary, out[1][t] = target logit.
// Two buffers alternate by epoch: a peer can only be one call ahead, because a call needs every rank's push.
__global__ void __launch_bounds__(kCeTpThreads)
ce_combine_tp_kernel(const float* __restrict__ parts, float* __restrict__ out, int T, int max_tokens, int rank, int tp,
                     uint32_t epoch, FuseArgs ptrs, int flags_per_src, int* __restrict__ err) {
  __shared__ int failed;
  const int t = blockIdx.x * kCeTpThreads + threadIdx.x;
  const size_t slot = (size_t)max_tokens * 3;
  const size_t par = (size_t)(epoch & 1) * tp * slot;
  float m = -INFINITY, s = 0.f, tl = 0.f;
  if (threadIdx.x == 0) failed = 0;
  if (t < T) {
    m = parts[(size_t)t * 3];
    s = parts[(size_t)t * 3 + 1];
    tl = parts[(size_t)t * 3 + 2];
    for (int p = 0; p < tp; ++p) {
      if (p == rank) continue;
      float* dst = reinterpret_cast<float*>(ptrs.data_ptrs[p]) + par + (size_t)rank * slot + (size_t)t * 3;
      dst[0] = m;
      dst[1] = s;
      dst[2] = tl;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int p = 0; p < tp; ++p)
      if (p != rank) st_release_sys(ptrs.flag_ptrs[p] + (size_t)rank * flags_per_src + blockIdx.x, epoch);
  }
  if ((int)threadIdx.x < tp && (int)threadIdx.x != rank) {
    volatile int never = 0;
    if (!wait_flag_ge(ptrs.flag_ptrs[rank] + (size_t)threadIdx.x * flags_per_src + blockIdx.x, epoch, &never)) {
      failed = 1;
      atomicCAS(err, 0, kErrCeExchange);
    }
  }
  __syncthreads();
  if (t >= T || failed) return;
  const float* mine = reinterpret_cast<const float*>(ptrs.data_ptrs[rank]) + par;
  float gm = -INFINITY, gs = 0.f, gt = 0.f;
  for (int p = 0; p < tp; ++p) {
    float pm = m, ps = s, pt = tl;
    if (p != rank) {
      const float* src = mine + (size_t)p * slot + (size_t)t * 3;
      pm = src[0];
      ps = src[1];
      pt = src[2];
    }
    gt += pt;
    if (pm > -INFINITY) {
      const float nm = fmaxf(gm, pm);
      gs = gs * __expf(gm - nm) + ps * __expf(pm - nm);
      gm = nm;
    }
  }
  out[t] = __logf(gs) + gm;
  out[(size_t)T + t] = gt;
}
}  // namespace ell

// parts [T, 3] of this rank -> out [2][T] = (lse, target logit) over all tp ranks.  bufs[r] / flags[r]: rank r's
// exchange buffer ([2][tp][max_tokens][3] floats) and flag words ([tp][flags_per_src]) as peer pointers.
ELL_API int ell_ce_combine_tp(const float* parts, float* out, int T, int max_tokens, int rank, int tp,
                              unsigned int epoch, void* const* bufs, void* const* flags, int* err,
                              cudaStream_t stream) {
  using namespace ell;
  if (T == 0) return 0;
  if (tp < 1 || tp > kMaxTp || T > max_tokens) return -2;
  const int blocks = (T + kCeTpThreads - 1) / kCeTpThreads;
  const int flags_per_src = 8192;
  if (blocks > flags_per_src) return -2;
  FuseArgs a{};
  for (int i = 0; i < tp; ++i) {
    a.data_ptrs[i] = (__nv_bfloat16*)bufs[i];
    a.flag_ptrs[i] = (uint32_t*)flags[i];
  }
  ce_combine_tp_kernel<<<blocks, kCeTpThreads, 0, stream>>>(parts, out, T, max_tokens, rank, tp, epoch, a, flags_per_src,
                                                           err);
  return launch_status();
}
