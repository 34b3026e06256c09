// The real-gated linear recurrent unit: a diagonal recurrence per channel with input-dependent decay.
//
//   r = sigmoid(gr + br),  i = sigmoid(gi + bi)        (gr, gi: the block-diagonal gate products of u, float32)
//   log a = c * r                                      (c = -8 softplus(lambda) per channel, from the host)
//   S_t = a S_(t-1) + sqrt(1 - a^2) * i * u            (S = 0 before a sequence's first token, no special first step)
//   out = S_t * gelu_tanh(y + by)                      (the other branch of the block, float32 pre-activation)
//
// Everything is float32; the state [slot][W] is read at a step's start and written at its end.  A recurrence
// S_t = a_t S_(t-1) + b_t composes: (a, b) then (a', b') is (a a', a' b + b').  Prompt steps use that in two passes over
// segments of RG_SEG consecutive tokens of the step (a block owns 32 channels of one segment, a lane a channel, a warp a run of
// RG_RUN tokens): the first composes every segment into one map, the second folds the maps before a segment in a fixed
// order and walks the segment from the state that gives.  A sequence's first token of the step is the constant map that
// starts from the state the sequence left, so segments may hold the ends and starts of several sequences.  Steps of one
// token a sequence use a thread per (sequence, channel).
#include "common.cuh"

namespace edgelm {

constexpr int RG_RUN = 8, RG_WARPS = 8, RG_SEG = RG_RUN * RG_WARPS;

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

// One run of RG_RUN tokens of one channel, from the step's first token `first` on: decay and input of every token.  A
// sequence's first token of the step takes the state that the sequence left (`from` [seq][W]) instead of its neighbour's:
// it is the constant map (0, a S_left + b).  `last`: bit j says that token j ends its sequence's part of the step.
__device__ __forceinline__ void rglru_run(const float* __restrict__ gates, int ldg, const float* __restrict__ u, int ldu, float cc, float cbr,
                                          float cbi, const float* __restrict__ from, bool from_slots, const int32_t* __restrict__ seq_tok0,
                                          const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ tok_seq, int first, int n_tokens,
                                          int W, int ch, bool live, float* a, float* b, unsigned* last, float* keep) {
  *last = 0;
#pragma unroll
  for (int j = 0; j < RG_RUN; ++j) {
    a[j] = 1.f;
    b[j] = 0.f;
    const int t = first + j;
    if (live && t < n_tokens) {
      rglru_terms(gates[(size_t)t * ldg + ch] + cbr, gates[(size_t)t * ldg + W + ch] + cbi, u[(size_t)t * ldu + ch], cc, &a[j], &b[j]);
      const int s = tok_seq[t];
      if (t == seq_tok0[s]) {
        const float v = from[(size_t)(from_slots ? seq_slot[s] : s) * W + ch];
        if (keep) keep[(size_t)s * W + ch] = v;
        b[j] = fmaf(a[j], v, b[j]);
        a[j] = 0.f;
      }
      if (t + 1 == seq_tok0[s + 1]) *last |= 1u << j;
    }
  }
}

// Prompt steps, first pass: block (channels, segment) composes its RG_SEG tokens into one map (A, B) per channel,
// seg [segment][2][W], and keeps the states that the step's sequences start from, init [seq][W].
__global__ void __launch_bounds__(RG_WARPS * 32)
rglru_compose_kernel(const float* __restrict__ gates, int ldg, const float* __restrict__ br, const float* __restrict__ bi,
                     const float* __restrict__ u, int ldu, const float* __restrict__ c, const float* __restrict__ state,
                     float* __restrict__ seg, float* __restrict__ init, const int32_t* __restrict__ seq_tok0,
                     const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ tok_seq, int n_tokens, int W) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float runA[RG_WARPS][32], runB[RG_WARPS][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = blockIdx.x * 32 + lane, g = blockIdx.y;
  const bool live = ch < W;
  float a[RG_RUN], b[RG_RUN];
  unsigned last;
  rglru_run(gates, ldg, u, ldu, live ? c[ch] : 0.f, live ? br[ch] : 0.f, live ? bi[ch] : 0.f, state, true, seq_tok0, seq_slot, tok_seq,
            g * RG_SEG + warp * RG_RUN, n_tokens, W, ch, live, a, b, &last, init);
  float A = 1.f, B = 0.f;
#pragma unroll
  for (int j = 0; j < RG_RUN; ++j) {
    A *= a[j];
    B = fmaf(a[j], B, b[j]);
  }
  runA[warp][lane] = A;
  runB[warp][lane] = B;
  __syncthreads();
  if (warp == 0 && live) {
    A = 1.f, B = 0.f;
#pragma unroll
    for (int w = 0; w < RG_WARPS; ++w) {
      A *= runA[w][lane];
      B = fmaf(runA[w][lane], B, runB[w][lane]);
    }
    seg[((size_t)g * 2) * W + ch] = A;
    seg[((size_t)g * 2 + 1) * W + ch] = B;
  }
}

// Second pass: the state before the block's segment is the fold of the segments before it, in order (the step's first
// token starts a sequence, so the fold starts from anything); the block walks its tokens from there, writes the outputs
// and, at a sequence's last token, its state.
template <typename TO>
__global__ void __launch_bounds__(RG_WARPS * 32)
rglru_walk_kernel(const float* __restrict__ gates, int ldg, const float* __restrict__ br, const float* __restrict__ bi,
                  const float* __restrict__ u, int ldu, const float* __restrict__ c, const float* __restrict__ y, int ldy,
                  const float* __restrict__ by, const float* __restrict__ seg, const float* __restrict__ init, float* __restrict__ state,
                  TO* __restrict__ out, const int32_t* __restrict__ seq_tok0, const int32_t* __restrict__ seq_slot,
                  const int32_t* __restrict__ tok_seq, int n_tokens, int W) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float runA[RG_WARPS][32], runB[RG_WARPS][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = blockIdx.x * 32 + lane, g = blockIdx.y;
  const bool live = ch < W;
  const int first = g * RG_SEG + warp * RG_RUN;
  const float cby = live ? by[ch] : 0.f;
  float yv[RG_RUN];          // the other branch's values, asked for before the arithmetic that they do not enter
#pragma unroll
  for (int j = 0; j < RG_RUN; ++j) yv[j] = (live && first + j < n_tokens) ? y[(size_t)(first + j) * ldy + ch] : 0.f;
  float S = 0.f;
  if (live)
    for (int p = 0; p < g; ++p) S = fmaf(seg[((size_t)p * 2) * W + ch], S, seg[((size_t)p * 2 + 1) * W + ch]);
  float a[RG_RUN], b[RG_RUN];
  unsigned last;
  rglru_run(gates, ldg, u, ldu, live ? c[ch] : 0.f, live ? br[ch] : 0.f, live ? bi[ch] : 0.f, init, false, seq_tok0, seq_slot, tok_seq,
            first, n_tokens, W, ch, live, a, b, &last, nullptr);
  float A = 1.f, B = 0.f;
#pragma unroll
  for (int j = 0; j < RG_RUN; ++j) {
    A *= a[j];
    B = fmaf(a[j], B, b[j]);
  }
  runA[warp][lane] = A;
  runB[warp][lane] = B;
  __syncthreads();
  for (int w = 0; w < warp; ++w) S = fmaf(runA[w][lane], S, runB[w][lane]);
#pragma unroll
  for (int j = 0; j < RG_RUN; ++j) {
    const int t = first + j;
    S = fmaf(a[j], S, b[j]);
    if (live && t < n_tokens) {
      out[(size_t)t * W + ch] = from_f32<TO>(S * gelu_tanh_f(yv[j] + cby));
      if (last >> j & 1) state[(size_t)seq_slot[tok_seq[t]] * W + ch] = S;
    }
  }
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
// `single`: every sequence brings one token (token t is sequence t).  Otherwise `tok_seq` [tokens] names every token's
// sequence and `scratch` holds (n_seqs + 2 * segments) * W floats, segments = ceil(tokens / RG_SEG).
extern "C" int edgelm_rglru_scan(const float* gates, int ldg, const float* br, const float* bi, const float* u, int ldu, const float* c,
                                 const float* y, int ldy, const float* by, float* state, void* out, int out_dtype,
                                 const int32_t* seq_tok0, const int32_t* seq_slot, const int32_t* tok_seq, float* scratch, int n_seqs,
                                 int n_tokens, int W, int single, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  EL_REFUSE(n_tokens > 0 && n_seqs > 0 && W > 0 && ldg >= 2 * W && ldu >= W && ldy >= W, "rglru_scan: bad sizes (width %d)", W);
  EL_REFUSE(out_dtype == DT_F32 || out_dtype == DT_BF16, "rglru_scan: unknown dtype code %d", out_dtype);
  const int bit = pdl_bit_for_tokens(n_tokens);
  if (single) {
    EL_REFUSE(n_tokens == n_seqs && n_tokens <= 65535, "rglru_scan: a step of single tokens has as many tokens as sequences");
    const dim3 grid((W + 127) / 128, n_tokens), block(128);
    if (out_dtype == DT_F32) launch_pdl(bit, rglru_step_kernel<float>, grid, block, (size_t)0, stream, gates, ldg, br, bi, u, ldu, c, y, ldy, by, state, (float*)out, seq_slot, W);
    else launch_pdl(bit, rglru_step_kernel<__nv_bfloat16>, grid, block, (size_t)0, stream, gates, ldg, br, bi, u, ldu, c, y, ldy, by, state, (__nv_bfloat16*)out, seq_slot, W);
  } else {
    const int segs = (n_tokens + RG_SEG - 1) / RG_SEG;
    EL_REFUSE(tok_seq != nullptr && scratch != nullptr && segs <= 65535, "rglru_scan: a prompt step needs the tokens' sequences and scratch (%d segments)", segs);
    float* init = scratch;
    float* seg = scratch + (size_t)n_seqs * W;
    const dim3 grid((W + 31) / 32, segs), block(RG_WARPS * 32);
    launch_pdl(bit, rglru_compose_kernel, grid, block, (size_t)0, stream, gates, ldg, br, bi, u, ldu, c, (const float*)state, seg, init, seq_tok0, seq_slot, tok_seq, n_tokens, W);
    if (out_dtype == DT_F32) launch_pdl(bit, rglru_walk_kernel<float>, grid, block, (size_t)0, stream, gates, ldg, br, bi, u, ldu, c, y, ldy, by, (const float*)seg, (const float*)init, state, (float*)out, seq_tok0, seq_slot, tok_seq, n_tokens, W);
    else launch_pdl(bit, rglru_walk_kernel<__nv_bfloat16>, grid, block, (size_t)0, stream, gates, ldg, br, bi, u, ldu, c, y, ldy, by, (const float*)seg, (const float*)init, state, (__nv_bfloat16*)out, seq_tok0, seq_slot, tok_seq, n_tokens, W);
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
