// Fused Adam(W) on flat fp32 partitions + squared-norm reduction, for sm_100a.
//
// One pass over (master, grad, m, v) updates the fp32 master weights and moments and writes
// the bf16 working copy of the parameters, with the gradient un-scale / clip coefficient
// folded in.  This is the update step the ZeRO partition owner runs on its shard; it
// replaces apex multi_tensor_adam + the BF16 optimizer's separate fp32→bf16 copy
// (llm/utils/model/optimizer_helper.py:87-89).  HBM-bound: 16 B read + 12 B (+2 B) written
// per element.
#include "common.cuh"

namespace ell {

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2, grad_scale;
  int adamw;
};

// `scale_ptr` (optional, device) multiplies grad_scale: lets the clip coefficient computed
// on the device feed the update without a host round trip.
__global__ void adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                            float* __restrict__ v, __nv_bfloat16* __restrict__ p_lowp, long long n, AdamArgs a,
                            const float* __restrict__ scale_ptr) {
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
    if (p_lowp) {
      reinterpret_cast<__nv_bfloat162*>(p_lowp)[2 * i] = __floats2bfloat162_rn(pp.x, pp.y);
      reinterpret_cast<__nv_bfloat162*>(p_lowp)[2 * i + 1] = __floats2bfloat162_rn(pp.z, pp.w);
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long j = nv * 4 + threadIdx.x;
    float gr = g[j] * gs;
    if (!a.adamw) gr += a.weight_decay * p[j];
    float mj = a.beta1 * m[j] + (1.f - a.beta1) * gr;
    float vj = a.beta2 * v[j] + (1.f - a.beta2) * gr * gr;
    float upd = (mj / a.bias_c1) / (sqrtf(vj / a.bias_c2) + a.eps);
    if (a.adamw) upd += a.weight_decay * p[j];
    float pj = p[j] - a.lr * upd;
    p[j] = pj; m[j] = mj; v[j] = vj;
    if (p_lowp) p_lowp[j] = __float2bfloat16_rn(pj);
  }
}

// out[0] += sum(x^2) (fp32 atomics on one word per CTA); caller zeroes out[0].
__global__ void sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[33];
  float s = 0.f;
  const long long nv = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float4 t = reinterpret_cast<const float4*>(x)[i];
    s += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    float t = x[nv * 4 + threadIdx.x];
    s += t * t;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

}  // namespace ell

using namespace ell;

ELL_API int ell_adam(float* p, const float* g, float* m, float* v, void* p_lowp, long long n, float lr, float beta1,
                     float beta2, float eps, float weight_decay, float bias_c1, float bias_c2, float grad_scale,
                     int adamw, const float* scale_ptr, cudaStream_t stream) {
  if (n == 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2, grad_scale, adamw};
  long long blocks = (n / 4 + 255) / 256;
  int grid = (int)(blocks < 1 ? 1 : (blocks < kNumSMs * 16 ? blocks : kNumSMs * 16));
  adam_kernel<<<grid, 256, 0, stream>>>(p, g, m, v, (__nv_bfloat16*)p_lowp, n, a, scale_ptr);
  return launch_status();
}

ELL_API int ell_sumsq(const float* x, long long n, float* out, cudaStream_t stream) {
  if (n == 0) return 0;
  long long blocks = (n / 4 + 255) / 256;
  int grid = (int)(blocks < 1 ? 1 : (blocks < kNumSMs * 8 ? blocks : kNumSMs * 8));
  sumsq_kernel<<<grid, 256, 0, stream>>>(x, n, out);
  return launch_status();
}

// Make `dev`'s primary context current on the calling thread.  Worker threads (for example the
// autograd engine's) may reach a launcher before any runtime call was made on them.
ELL_API int ell_set_device(int dev) { return (int)cudaSetDevice(dev); }
