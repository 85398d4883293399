// ZeRO-1/2 data-parallel step as two kernels that do their collective themselves over NVLink peer memory
// (every rank's flat fp32 gradient buffer and bf16 parameter buffer live in symmetric memory):
//
//   zero_reduce_scatter_kernel   grad_shard = (sum over ranks of grad[r][shard]) / dp, read straight from the
//                                peers' buffers with 16-byte loads, written into this rank's own buffer, and the
//                                sum of squares of the reduced shard (two ranges, for the global-norm rule that
//                                counts TP-replicated parameters once) accumulated in the same pass.
//   zero_adam_allgather_kernel   Adam(W) on the fp32 master shard, and the updated bf16 parameters stored into
//                                every rank's parameter buffer (the all-gather) in the same pass.
//
// Ordering between ranks is the caller's (stream-ordered collectives before / between / after the two launches);
// the kernels themselves never wait on a peer.
// Replaces DeepSpeed's ZeRO stage-1/2 reduce-scatter + fused Adam + all-gather that the reference relies on
// (configs/megatron/template.yaml:12-24, llm/runners/base_llm_runner.py:196-202).
#include "common.cuh"

namespace ell {

constexpr int kZeroMaxDp = 16;

struct ZeroPeers {
  const float* grad[kZeroMaxDp];
  __nv_bfloat16* param[kZeroMaxDp];
};

__global__ void __launch_bounds__(256)
zero_reduce_scatter_kernel(ZeroPeers peers, int dp, int rank, long long shard_lo, long long n, float inv_dp,
                           long long split, float* __restrict__ sumsq2) {
  __shared__ float red[33];
  float s_lo = 0.f, s_hi = 0.f;
  float* mine = const_cast<float*>(peers.grad[rank]) + shard_lo;
  const long long nv = n / 4;   // shard sizes are multiples of 4 by construction
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = reinterpret_cast<const float4*>(mine)[i];
#pragma unroll 1
    for (int k = 1; k < dp; ++k) {
      const int p = (rank + k) % dp;           // every rank starts at a different peer
      const float4 t = reinterpret_cast<const float4*>(peers.grad[p] + shard_lo)[i];
      acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    }
    acc.x *= inv_dp; acc.y *= inv_dp; acc.z *= inv_dp; acc.w *= inv_dp;
    reinterpret_cast<float4*>(mine)[i] = acc;
    const float sq = acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    if (shard_lo + i * 4 < split) s_lo += sq; else s_hi += sq;
  }
  s_lo = block_sum(s_lo, red);
  s_hi = block_sum(s_hi, red);
  if (threadIdx.x == 0) {
    if (s_lo != 0.f) atomicAdd(&sumsq2[0], s_lo);
    if (s_hi != 0.f) atomicAdd(&sumsq2[1], s_hi);
  }
}

struct ZeroAdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2, grad_scale;
  int adamw;
};

__global__ void __launch_bounds__(256)
zero_adam_allgather_kernel(ZeroPeers peers, int dp, int rank, long long off, long long n, float* __restrict__ p,
                           const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v, ZeroAdamArgs a,
                           const float* __restrict__ scale_ptr) {
  // `off` is the position of element 0 of p/g/m/v inside the flat parameter buffer of every rank
  const float gs = a.grad_scale * (scale_ptr ? *scale_ptr : 1.f);
  const long long nv = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i], gg = reinterpret_cast<const float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
    float* P = &pp.x; float* G = &gg.x; float* M = &mm.x; float* V = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gr = G[j] * gs;
      if (!a.adamw) gr += a.weight_decay * P[j];
      M[j] = a.beta1 * M[j] + (1.f - a.beta1) * gr;
      V[j] = a.beta2 * V[j] + (1.f - a.beta2) * gr * gr;
      float upd = (M[j] / a.bias_c1) / (sqrtf(V[j] / a.bias_c2) + a.eps);
      if (a.adamw) upd += a.weight_decay * P[j];
      P[j] -= a.lr * upd;
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
    const uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
#pragma unroll 1
    for (int k = 0; k < dp; ++k) {
      const int q = (rank + k) % dp;
      reinterpret_cast<uint2*>(peers.param[q] + off)[i] = packed;
    }
  }
}

}  // namespace ell

using namespace ell;

// grad_ptrs[r]: rank r's flat fp32 gradient buffer (peer pointers; entry `rank` is local).  Reduces elements
// [shard_lo, shard_lo + n) over the dp ranks into this rank's buffer (scaled by 1/dp) and adds the squared norm
// of the result to sumsq2[0] (elements below `split`) / sumsq2[1] (the rest); the caller zeroes sumsq2.
ELL_API int ell_zero_reduce_scatter(void* const* grad_ptrs, int dp, int rank, long long shard_lo, long long n,
                                    long long split, float* sumsq2, cudaStream_t stream) {
  if (n == 0) return 0;
  if (dp < 1 || dp > kZeroMaxDp || (n & 3) || (shard_lo & 3)) return -1;
  ZeroPeers peers{};
  for (int i = 0; i < dp; ++i) peers.grad[i] = (const float*)grad_ptrs[i];
  long long blocks = (n / 4 + 255) / 256;
  int grid = (int)(blocks < kNumSMs * 8 ? blocks : kNumSMs * 8);
  zero_reduce_scatter_kernel<<<grid, 256, 0, stream>>>(peers, dp, rank, shard_lo, n, 1.f / (float)dp, split, sumsq2);
  return launch_status();
}

// Adam(W) on n elements of the master shard (p, g, m, v point at the same shard-relative range), writing the
// bf16 parameters to param_ptrs[r] + off on every rank r.  n and off must be multiples of 4.
ELL_API int ell_zero_adam_allgather(void* const* param_ptrs, int dp, int rank, long long off, long long n, float* p,
                                    const float* g, float* m, float* v, float lr, float beta1, float beta2, float eps,
                                    float weight_decay, float bias_c1, float bias_c2, float grad_scale, int adamw,
                                    const float* scale_ptr, cudaStream_t stream) {
  if (n == 0) return 0;
  if (dp < 1 || dp > kZeroMaxDp || (n & 3) || (off & 3)) return -1;
  ZeroPeers peers{};
  for (int i = 0; i < dp; ++i) peers.param[i] = (__nv_bfloat16*)param_ptrs[i];
  ZeroAdamArgs a{lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2, grad_scale, adamw};
  long long blocks = (n / 4 + 255) / 256;
  int grid = (int)(blocks < kNumSMs * 8 ? blocks : kNumSMs * 8);
  zero_adam_allgather_kernel<<<grid, 256, 0, stream>>>(peers, dp, rank, off, n, p, g, m, v, a, scale_ptr);
  return launch_status();
}
