// The real-gated linear recurrent unit: a diagonal recurrence per channel with input-dependent decay.
//
//   r = sigmoid(gr + br),  i = sigmoid(gi + bi)        (gr, gi: the block-diagonal gate products of u, float32)
//   log a = c * r                                      (c = -8 softplus(lambda) per channel, from the host)
//   S_t = a S_(t-1) + sqrt(1 - a^2) * i * u            (S = 0 before a sequence's first token, no special first step)
//   out = S_t * gelu_tanh(y + by)                      (the other branch of the block, float32 pre-activation)
//
// Everything is float32; the state [slot][W] is read at a step's start and written at its end.  A recurrence
// S_t = a_t S_(t-1) + b_t composes: (a, b) then (a', b') is (a a', a' b + b').  Prompt steps use that: a block owns 32
// channels of one sequence (a lane a channel), its warps take runs of RG_RUN consecutive tokens each, compose their run from
// zero, fold the runs before theirs in a fixed order, and walk their run again from the state that gives.  Steps of one
// token a sequence use a thread per (sequence, channel).
#include "common.cuh"

namespace edgelm {

constexpr int RG_RUN = 8, RG_WARPS = 8;

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// decay and input of one (token, channel): a = exp(c r), b = sqrt(1 - a^2) i u, with 1 - a^2 = -expm1(2 c r)
__device__ __forceinline__ void rglru_terms(float gr, float gi, float u, float c, float* a, float* b) {
  const float la = c * sigmoid_f(gr);
  *a = expf(la);
  *b = sqrtf(-expm1f(2.0f * la)) * sigmoid_f(gi) * u;
}

template <typename TO>
__global__ void __launch_bounds__(RG_WARPS * 32)
rglru_scan_kernel(const float* __restrict__ gates, int ldg, const float* __restrict__ br, const float* __restrict__ bi,
                  const float* __restrict__ u, int ldu, const float* __restrict__ c, const float* __restrict__ y, int ldy,
                  const float* __restrict__ by, float* __restrict__ state, TO* __restrict__ out, const int32_t* __restrict__ seq_tok0,
                  const int32_t* __restrict__ seq_slot, int W) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float runA[RG_WARPS][32], runB[RG_WARPS][32], carry[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = blockIdx.x * 32 + lane, s = blockIdx.y;
  const bool live = ch < W;
  const int t0 = seq_tok0[s], n = seq_tok0[s + 1] - t0;
  float* st = state + (size_t)seq_slot[s] * W;
  const float cc = live ? c[ch] : 0.f, cbr = live ? br[ch] : 0.f, cbi = live ? bi[ch] : 0.f, cby = live ? by[ch] : 0.f;
  if (warp == 0) carry[lane] = live ? st[ch] : 0.f;
  __syncthreads();
  for (int base = 0; base < n; base += RG_WARPS * RG_RUN) {
    const int first = base + warp * RG_RUN;
    float a[RG_RUN], b[RG_RUN];
    float A = 1.f, B = 0.f;
#pragma unroll
    for (int j = 0; j < RG_RUN; ++j) {
      a[j] = 1.f;
      b[j] = 0.f;
      if (live && first + j < n) {
        const size_t t = (size_t)(t0 + first + j);
        rglru_terms(gates[t * ldg + ch] + cbr, gates[t * ldg + W + ch] + cbi, u[t * ldu + ch], cc, &a[j], &b[j]);
      }
      A *= a[j];
      B = fmaf(a[j], B, b[j]);
    }
    runA[warp][lane] = A;
    runB[warp][lane] = B;
    __syncthreads();
    float S = carry[lane];
    for (int w = 0; w < warp; ++w) S = fmaf(runA[w][lane], S, runB[w][lane]);
#pragma unroll
    for (int j = 0; j < RG_RUN; ++j) {
      S = fmaf(a[j], S, b[j]);
      if (live && first + j < n) {
        const size_t t = (size_t)(t0 + first + j);
        out[t * W + ch] = from_f32<TO>(S * gelu_tanh_f(y[t * ldy + ch] + cby));
      }
    }
    __syncthreads();                       // every warp has read the carry and the runs
    if (warp == RG_WARPS - 1) carry[lane] = S;    // (runs past the sequence's end are the identity)
    __syncthreads();
  }
  if (warp == 0 && live) st[ch] = carry[lane];
}

template <typename TO>
__global__ void rglru_step_kernel(const float* __restrict__ gates, int ldg, const float* __restrict__ br, const float* __restrict__ bi,
                                  const float* __restrict__ u, int ldu, const float* __restrict__ c, const float* __restrict__ y, int ldy,
                                  const float* __restrict__ by, float* __restrict__ state, TO* __restrict__ out,
                                  const int32_t* __restrict__ seq_slot, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y, ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= W) return;
  float* st = state + (size_t)seq_slot[t] * W;
  float a, b;
  rglru_terms(gates[(size_t)t * ldg + ch] + br[ch], gates[(size_t)t * ldg + W + ch] + bi[ch], u[(size_t)t * ldu + ch], c[ch], &a, &b);
  const float S = fmaf(a, st[ch], b);
  st[ch] = S;
  out[(size_t)t * W + ch] = from_f32<TO>(S * gelu_tanh_f(y[(size_t)t * ldy + ch] + by[ch]));
}

// mid = g sigmoid(alpha g) (v + 1) with g = min(gate, limit), v = clamp(up, -limit, limit); gu [tokens][2 F] float32 = gate | up
template <typename TO>
__global__ void clamped_glu_kernel(const float* __restrict__ gu, TO* __restrict__ mid, int F, float limit, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  const float* row = gu + (size_t)blockIdx.x * 2 * F;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float g = fminf(row[i], limit), v = fminf(fmaxf(row[F + i], -limit), limit);
    mid[(size_t)blockIdx.x * F + i] = from_f32<TO>(g * sigmoid_f(alpha * g) * (v + 1.0f));
  }
}

}  // namespace edgelm

using namespace edgelm;

// gates [tokens][>= 2 W] (r | i pre-activations, row pitch ldg), u [tokens][W..] (pitch ldu), y [tokens][W..] (pitch ldy);
// `single`: every sequence brings one token (token t is sequence t).
extern "C" int edgelm_rglru_scan(const float* gates, int ldg, const float* br, const float* bi, const float* u, int ldu, const float* c,
                                 const float* y, int ldy, const float* by, float* state, void* out, int out_dtype,
                                 const int32_t* seq_tok0, const int32_t* seq_slot, int n_seqs, int n_tokens, int W, int single,
                                 cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  EL_REFUSE(n_tokens > 0 && n_seqs > 0 && W > 0 && ldg >= 2 * W && ldu >= W && ldy >= W && n_seqs <= 65535, "rglru_scan: bad sizes (width %d)", W);
  EL_REFUSE(out_dtype == DT_F32 || out_dtype == DT_BF16, "rglru_scan: unknown dtype code %d", out_dtype);
  const int bit = pdl_bit_for_tokens(n_tokens);
  if (single) {
    EL_REFUSE(n_tokens == n_seqs, "rglru_scan: a step of single tokens has as many tokens as sequences");
    const dim3 grid((W + 127) / 128, n_tokens), block(128);
    if (out_dtype == DT_F32) launch_pdl(bit, rglru_step_kernel<float>, grid, block, (size_t)0, stream, gates, ldg, br, bi, u, ldu, c, y, ldy, by, state, (float*)out, seq_slot, W);
    else launch_pdl(bit, rglru_step_kernel<__nv_bfloat16>, grid, block, (size_t)0, stream, gates, ldg, br, bi, u, ldu, c, y, ldy, by, state, (__nv_bfloat16*)out, seq_slot, W);
  } else {
    const dim3 grid((W + 31) / 32, n_seqs), block(RG_WARPS * 32);
    if (out_dtype == DT_F32) launch_pdl(bit, rglru_scan_kernel<float>, grid, block, (size_t)0, stream, gates, ldg, br, bi, u, ldu, c, y, ldy, by, state, (float*)out, seq_tok0, seq_slot, W);
    else launch_pdl(bit, rglru_scan_kernel<__nv_bfloat16>, grid, block, (size_t)0, stream, gates, ldg, br, bi, u, ldu, c, y, ldy, by, state, (__nv_bfloat16*)out, seq_tok0, seq_slot, W);
  }
  EL_LAUNCH_CHECK("rglru_scan");
  return 0;
}

extern "C" int edgelm_clamped_glu(const float* gu, void* mid, int out_dtype, int n_tokens, int F, float limit, float alpha, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && F > 0 && limit > 0.f, "clamped_glu: bad sizes");
  const dim3 grid(n_tokens), block(F >= 1024 ? 256 : 128);
  const int bit = pdl_bit_for_tokens(n_tokens);
  if (out_dtype == DT_F32) launch_pdl(bit, clamped_glu_kernel<float>, grid, block, (size_t)0, stream, gu, (float*)mid, F, limit, alpha);
  else if (out_dtype == DT_BF16) launch_pdl(bit, clamped_glu_kernel<__nv_bfloat16>, grid, block, (size_t)0, stream, gu, (__nv_bfloat16*)mid, F, limit, alpha);
  else EL_REFUSE(false, "clamped_glu: unknown dtype code %d", out_dtype);
  EL_LAUNCH_CHECK("clamped_glu");
  return 0;
}
