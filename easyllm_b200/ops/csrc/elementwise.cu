// RoPE and SwiGLU kernels for sm_100a (HBM-bound elementwise ops, 16-byte vector access).
//
// RoPE is applied in place on the q and k heads of the packed QKV GEMM output
// `[T, (Hq + 2·Hk) · D]` (NeoX half rotation, positions gathered per token so packed documents
// restart at 0).  The backward is the same rotation with -sin.  Replaces the eager /
// Triton rotary of the reference (llm/models/mg_models/llama/positional_embeddings.py:94-122).
//
// SwiGLU reads the fused gate|up GEMM output `[T, 2F]` (gate columns first) and writes
// `silu(gate) * up` `[T, F]`; the backward recomputes the activation from gate|up
// (llm/models/mg_models/llama/transformer.py:217-225 materialises both halves and the SiLU).
#include "common.cuh"

namespace ell {

// One thread rotates 8 (x1) + 8 (x2) elements of one head: D/2 must be a multiple of 8.
// A position outside the cos / sin tables is reported through the error word (code 32) and its row left unrotated,
// instead of reading past the tables.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ pos, int T, int row_stride,
                            int n_rot_heads, int D, float sin_sign, int table_rows, int* __restrict__ err) {
  const int half = D / 2, vec_per_head = half / 8;
  const long long total = (long long)T * n_rot_heads * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const int hd = (int)((i / vec_per_head) % n_rot_heads);
    const int t = (int)(i / ((long long)vec_per_head * n_rot_heads));
    const int p = pos[t];
    if (p < 0 || p >= table_rows) {
      if (err != nullptr) atomicCAS(err, 0, 32);
      continue;
    }
    __nv_bfloat16* base = qkv + (size_t)t * row_stride + (size_t)hd * D + v * 8;
    float x1[8], x2[8], c[8], s[8];
    unpack8(*reinterpret_cast<const bf16x8*>(base), x1);
    unpack8(*reinterpret_cast<const bf16x8*>(base + half), x2);
    const float4* cp = reinterpret_cast<const float4*>(cos_t + (size_t)p * half + v * 8);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + (size_t)p * half + v * 8);
    float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
    float o1[8], o2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sj = s[j] * sin_sign;
      o1[j] = x1[j] * c[j] - x2[j] * sj;
      o2[j] = x2[j] * c[j] + x1[j] * sj;
    }
    *reinterpret_cast<bf16x8*>(base) = pack8(o1);
    *reinterpret_cast<bf16x8*>(base + half) = pack8(o2);
  }
}

__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int T, int F) {
  const int fv = F / 8;
  const long long total = (long long)T * fv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / fv), c = (int)(i % fv);
    float g[8], u[8], o[8];
    unpack8(reinterpret_cast<const bf16x8*>(gu + (size_t)t * 2 * F)[c], g);
    unpack8(reinterpret_cast<const bf16x8*>(gu + (size_t)t * 2 * F + F)[c], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    reinterpret_cast<bf16x8*>(out + (size_t)t * F)[c] = pack8(o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, int T, int F) {
  const int fv = F / 8;
  const long long total = (long long)T * fv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / fv), c = (int)(i % fv);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(reinterpret_cast<const bf16x8*>(gu + (size_t)t * 2 * F)[c], g);
    unpack8(reinterpret_cast<const bf16x8*>(gu + (size_t)t * 2 * F + F)[c], u);
    unpack8(reinterpret_cast<const bf16x8*>(dout + (size_t)t * F)[c], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * sg * (1.f + g[j] * (1.f - sg));
    }
    reinterpret_cast<bf16x8*>(dgu + (size_t)t * 2 * F)[c] = pack8(dg);
    reinterpret_cast<bf16x8*>(dgu + (size_t)t * 2 * F + F)[c] = pack8(du);
  }
}

// out(fp32) += in(bf16): gradient accumulation of one parameter into the fp32 flat buffer.
__global__ void accum_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, long long n) {
  const long long nv = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(in)[i], f);
    float4* o = reinterpret_cast<float4*>(out) + 2 * i;
    float4 a = o[0], b = o[1];
    a.x += f[0]; a.y += f[1]; a.z += f[2]; a.w += f[3];
    b.x += f[4]; b.y += f[5]; b.z += f[6]; b.w += f[7];
    o[0] = a; o[1] = b;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    const long long j = nv * 8 + threadIdx.x;
    out[j] += __bfloat162float(in[j]);
  }
}

inline int ew_grid(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  long long cap = (long long)kNumSMs * 16;
  return (int)(b < 1 ? 1 : (b < cap ? b : cap));
}

}  // namespace ell

using namespace ell;

// cos_t / sin_t: fp32 [table_rows, D/2]; positions outside [0, table_rows) set *err to 32.
ELL_API int ell_rope(void* qkv, const float* cos_t, const float* sin_t, const int* pos, int T, int row_stride,
                     int n_rot_heads, int D, int backward, int table_rows, int* err, cudaStream_t stream) {
  if (D % 16) return -1;
  long long total = (long long)T * n_rot_heads * (D / 16);
  if (total == 0) return 0;
  rope_kernel<<<ew_grid(total, 256), 256, 0, stream>>>((__nv_bfloat16*)qkv, cos_t, sin_t, pos, T, row_stride,
                                                       n_rot_heads, D, backward ? -1.f : 1.f, table_rows, err);
  return launch_status();
}

ELL_API int ell_swiglu_fwd(const void* gu, void* out, int T, int F, cudaStream_t stream) {
  if (F % 8) return -1;
  long long total = (long long)T * (F / 8);
  if (total == 0) return 0;
  swiglu_fwd_kernel<<<ew_grid(total, 256), 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, F);
  return launch_status();
}

ELL_API int ell_swiglu_bwd(const void* dout, const void* gu, void* dgu, int T, int F, cudaStream_t stream) {
  if (F % 8) return -1;
  long long total = (long long)T * (F / 8);
  if (total == 0) return 0;
  swiglu_bwd_kernel<<<ew_grid(total, 256), 256, 0, stream>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)gu,
                                                            (__nv_bfloat16*)dgu, T, F);
  return launch_status();
}

ELL_API int ell_accum_bf16_to_f32(const void* in, float* out, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  accum_bf16_to_f32_kernel<<<ew_grid(n / 8 + 1, 256), 256, 0, stream>>>((const __nv_bfloat16*)in, out, n);
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// Vocab-parallel embedding: masked row gather, and its backward as an fp32 scatter-add straight
// into the weight's gradient accumulator (no bf16 gradient tensor, no sort).
// Replaces F.embedding + mask writes of the reference
// (llm/models/mg_models/base_modules/layers/vocab_parallel_emb.py:106-137).
// ---------------------------------------------------------------------------------------------
namespace ell {

// out[t, :] = ids[t] in [vocab_start, vocab_start + rows) ? weight[ids[t] - vocab_start, :] : 0
// An id outside [0, vocab_total) is reported through the error word (code 31) instead of a host-side max() of the
// ids, which would cost a device synchronisation per micro-batch; its row is written as zeros.
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ weight,
                                     __nv_bfloat16* __restrict__ out, int T, int cols, long long vocab_start,
                                     long long rows, long long vocab_total, int* __restrict__ err) {
  const int nvec = cols / 8;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const long long id = ids[t];
    if (err != nullptr && threadIdx.x == 0 && (id < 0 || id >= vocab_total)) atomicCAS(err, 0, 31);
    const long long loc = id - vocab_start;
    const bool mine = loc >= 0 && loc < rows;
    const bf16x8* src = reinterpret_cast<const bf16x8*>(weight + (mine ? loc : 0) * cols);
    bf16x8* dst = reinterpret_cast<bf16x8*>(out + (size_t)t * cols);
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) dst[c] = mine ? src[c] : bf16x8{};
  }
}

// grad32[ids[t] - vocab_start, :] += dout[t, :] for the ids this rank owns (fp32 vector atomics)
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ grad32, int T, int cols, long long vocab_start,
                                     long long rows) {
  const int nvec = cols / 8;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const long long loc = ids[t] - vocab_start;
    if (loc < 0 || loc >= rows) continue;
    const bf16x8* src = reinterpret_cast<const bf16x8*>(dout + (size_t)t * cols);
    float* dst = grad32 + loc * cols;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      float f[8];
      unpack8(src[c], f);
      atomicAdd(reinterpret_cast<float4*>(dst + c * 8), make_float4(f[0], f[1], f[2], f[3]));
      atomicAdd(reinterpret_cast<float4*>(dst + c * 8 + 4), make_float4(f[4], f[5], f[6], f[7]));
    }
  }
}

}  // namespace ell

// vocab_total > 0 with err != nullptr: ids outside [0, vocab_total) set *err to 31.
ELL_API int ell_embedding_fwd(const long long* ids, const void* weight, void* out, int T, int cols,
                              long long vocab_start, long long rows, long long vocab_total, int* err,
                              cudaStream_t stream) {
  if (T == 0) return 0;
  if (cols % 8) return -1;
  const int grid = T < ell::kNumSMs * 16 ? T : ell::kNumSMs * 16;
  ell::embedding_fwd_kernel<<<grid, 128, 0, stream>>>(ids, (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, T, cols,
                                                       vocab_start, rows, vocab_total, vocab_total > 0 ? err : nullptr);
  return ell::launch_status();
}

ELL_API int ell_embedding_bwd(const long long* ids, const void* dout, float* grad32, int T, int cols,
                              long long vocab_start, long long rows, cudaStream_t stream) {
  if (T == 0) return 0;
  if (cols % 8) return -1;
  const int grid = T < ell::kNumSMs * 16 ? T : ell::kNumSMs * 16;
  ell::embedding_bwd_kernel<<<grid, 128, 0, stream>>>(ids, (const __nv_bfloat16*)dout, grad32, T, cols, vocab_start,
                                                       rows);
  return ell::launch_status();
}

namespace ell {
// Column sums of a bf16 matrix added into fp32: out[c] += sum_r x[r, c].  The bias gradient of a linear layer
// (db = sum over tokens of dy) without materialising an fp32 copy of dy.  A block covers 256 columns (32 threads x 8
// columns, 16-byte loads) and a slice of the rows (8 row lanes); lanes meet in shared memory, one atomic per column
// and block.
__global__ void __launch_bounds__(256) colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out,
                                                     int rows, int cols) {
  __shared__ float red[8][256];
  const int cg = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 256 + cg * 8;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  if (c0 < cols) {
    for (int r = blockIdx.y * 8 + rl; r < rows; r += gridDim.y * 8) {
      float t[8];
      unpack8(*reinterpret_cast<const bf16x8*>(x + (size_t)r * cols + c0), t);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += t[e];
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[rl][cg * 8 + e] = acc[e];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < cols) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red[i][threadIdx.x];
    atomicAdd(out + c, s);
  }
}
}  // namespace ell

// out[cols] (fp32) += column sums of x[rows, cols] (bf16, cols a multiple of 8).
ELL_API int ell_colsum_bf16(const void* x, float* out, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 8) return -1;
  const int bx = (cols + 255) / 256;
  int by = (rows + 63) / 64;
  const int cap = (ell::kNumSMs * 8 + bx - 1) / bx;
  if (by > cap) by = cap;
  if (by < 1) by = 1;
  ell::colsum_kernel<<<dim3(bx, by), 256, 0, stream>>>((const __nv_bfloat16*)x, out, rows, cols);
  return ell::launch_status();
}
