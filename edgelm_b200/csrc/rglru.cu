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
// RG_RUN tokens): the first turns gates into decays and inputs and composes every segment into one map, the second folds the
// maps before a segment in a fixed order and walks the segment from the state that gives.  A sequence's first token of the step is the constant map that
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

// Prompt steps, first pass: block (channels, segment) turns the gates of its RG_SEG tokens into decay and input, IN PLACE
// (gates[t][ch] <- a, gates[t][W + ch] <- b), and composes them into one map (A, B) per channel, seg [segment][2][W].  A
// sequence's first token of the step takes the state that the sequence left instead of its neighbour's: it becomes the
// constant map (0, a S_left + b).
__global__ void __launch_bounds__(RG_WARPS * 32)
rglru_compose_kernel(float* __restrict__ gates, int ldg, const float* __restrict__ br, const float* __restrict__ bi,
                     const float* __restrict__ u, int ldu, const float* __restrict__ c, const float* __restrict__ state,
                     float* __restrict__ seg, const int32_t* __restrict__ seq_tok0, const int32_t* __restrict__ seq_slot,
                     const int32_t* __restrict__ tok_seq, int n_tokens, int W) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float runA[RG_WARPS][32], runB[RG_WARPS][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = blockIdx.x * 32 + lane, g = blockIdx.y;
  const bool live = ch < W;
  const int first = g * RG_SEG + warp * RG_RUN;
  const float cc = live ? c[ch] : 0.f, cbr = live ? br[ch] : 0.f, cbi = live ? bi[ch] : 0.f;
  float gr[RG_RUN], gi[RG_RUN], uv[RG_RUN];
#pragma unroll
  for (int j = 0; j < RG_RUN; ++j) {           // (all loads first: they do not depend on one another)
    const bool on = live && first + j < n_tokens;
    const size_t t = (size_t)(first + j);
    gr[j] = on ? gates[t * ldg + ch] : 0.f;
    gi[j] = on ? gates[t * ldg + W + ch] : 0.f;
    uv[j] = on ? u[t * ldu + ch] : 0.f;
  }
  float A = 1.f, B = 0.f;
#pragma unroll
  for (int j = 0; j < RG_RUN; ++j) {
    const int t = first + j;
    if (live && t < n_tokens) {
      float a, b;
      rglru_terms(gr[j] + cbr, gi[j] + cbi, uv[j], cc, &a, &b);
      const int s = tok_seq[t];
      if (t == seq_tok0[s]) {
        b = fmaf(a, state[(size_t)seq_slot[s] * W + ch], b);
        a = 0.f;
      }
      gates[(size_t)t * ldg + ch] = a;
      gates[(size_t)t * ldg + W + ch] = b;
      A *= a;
      B = fmaf(a, B, b);
    }
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

// Second pass, over ab [tokens][2 W] = decays | inputs as the first left them: the state before the block's segment is the
// fold of the segments before it, in order (the step's first token starts a sequence, so the fold may start from anything);
// the block walks its tokens from there, writes the outputs and, at a sequence's last token, its state.
template <typename TO>
__global__ void __launch_bounds__(RG_WARPS * 32)
rglru_walk_kernel(const float* __restrict__ ab, int ldg, const float* __restrict__ y, int ldy, const float* __restrict__ by,
                  const float* __restrict__ seg, float* __restrict__ state, TO* __restrict__ out, const int32_t* __restrict__ seq_tok0,
                  const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ tok_seq, int n_tokens, int W) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float runA[RG_WARPS][32], runB[RG_WARPS][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = blockIdx.x * 32 + lane, g = blockIdx.y;
  const bool live = ch < W;
  const int first = g * RG_SEG + warp * RG_RUN;
  const float cby = live ? by[ch] : 0.f;
  float a[RG_RUN], b[RG_RUN], yv[RG_RUN];
#pragma unroll
  for (int j = 0; j < RG_RUN; ++j) {
    const bool on = live && first + j < n_tokens;
    const size_t t = (size_t)(first + j);
    a[j] = on ? ab[t * ldg + ch] : 1.f;
    b[j] = on ? ab[t * ldg + W + ch] : 0.f;
    yv[j] = on ? y[t * ldy + ch] : 0.f;
  }
  float S = 0.f;
  if (live)
    for (int p = 0; p < g; ++p) S = fmaf(seg[((size_t)p * 2) * W + ch], S, seg[((size_t)p * 2 + 1) * W + ch]);
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
      const int s = tok_seq[t];
      if (t + 1 == seq_tok0[s + 1]) state[(size_t)seq_slot[s] * W + ch] = S;
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

// The gates' products on the tensor cores, exact to float32: gates[t][b bw + n] = sum_k ra[b][n][k] u[t][b bw + k] and the same
// with ri into the second half of the row.  The weights are bfloat16; a float32 input is the sum of three bfloat16 terms
// (8 + 8 + 8 bits of its 24), every product of a term and a weight is exact in float32, and the sums are float32: the
// result differs from the float32 product by the order of the sums only.  A block takes 64 tokens x 32 columns of both
// matrices of one diagonal block (they share the staged input), a warp 16 tokens, K in chunks of 32.
constexpr int GT_M = 64, GT_N = 32, GT_KC = 32, GT_LD = GT_KC + 8;      // (rows of 40 bfloat16: fragment reads hit 32 banks)

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(__nv_bfloat16 lo, __nv_bfloat16 hi) {
  return (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
}

__global__ void __launch_bounds__(128, 4)
rglru_gates_mma_kernel(const float* __restrict__ u, int ldu, const __nv_bfloat16* __restrict__ w_ra, const __nv_bfloat16* __restrict__ w_ri,
                       float* __restrict__ gates, int ldg, int n_tokens, int W, int bw) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ __align__(16) __nv_bfloat16 As[3][GT_M][GT_LD];
  __shared__ __align__(16) __nv_bfloat16 Ws[2 * GT_N][GT_LD];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gq = lane >> 2, cq = lane & 3;
  const int t0 = blockIdx.x * GT_M, n0 = blockIdx.y * GT_N, blk = blockIdx.z;
  const float* ub = u + (size_t)blk * bw;
  float acc[8][4] = {};
  // a chunk's global loads are issued a chunk ahead, into registers, and reach shared memory (the input split into its three
  // terms on the way) when the chunk before has been multiplied: the loads' latency hides behind those multiply-adds
  constexpr int A_IT = GT_M * (GT_KC / 2) / 128, W_IT = 2 * GT_N * GT_KC / 128;
  float xa[A_IT][2];
  __nv_bfloat16 xw[W_IT];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int it = 0; it < A_IT; ++it) {
      const int i = threadIdx.x + it * 128, r = i / (GT_KC / 2), k = (i - r * (GT_KC / 2)) * 2;
      const bool row = t0 + r < n_tokens;
#pragma unroll
      for (int e = 0; e < 2; ++e) xa[it][e] = (row && k0 + k + e < bw) ? ub[(size_t)(t0 + r) * ldu + k0 + k + e] : 0.f;
    }
#pragma unroll
    for (int it = 0; it < W_IT; ++it) {      // rows n0 .. n0 + 31 of ra[blk], then of ri[blk]
      const int i = threadIdx.x + it * 128, r = i / GT_KC, k = i - r * GT_KC, n = n0 + (r % GT_N);
      const __nv_bfloat16* wm = r < GT_N ? w_ra : w_ri;
      xw[it] = (n < bw && k0 + k < bw) ? wm[((size_t)blk * bw + n) * bw + k0 + k] : __float2bfloat16(0.f);
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < bw; k0 += GT_KC) {
#pragma unroll
    for (int it = 0; it < A_IT; ++it) {
      const int i = threadIdx.x + it * 128, r = i / (GT_KC / 2), k = (i - r * (GT_KC / 2)) * 2;
      __nv_bfloat16 p[3][2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float rest = xa[it][e];
#pragma unroll
        for (int q = 0; q < 3; ++q) {
          p[q][e] = __float2bfloat16(rest);
          rest -= __bfloat162float(p[q][e]);
        }
      }
#pragma unroll
      for (int q = 0; q < 3; ++q) *reinterpret_cast<uint32_t*>(&As[q][r][k]) = pack_bf16(p[q][0], p[q][1]);
    }
#pragma unroll
    for (int it = 0; it < W_IT; ++it) {
      const int i = threadIdx.x + it * 128, r = i / GT_KC, k = i - r * GT_KC;
      Ws[r][k] = xw[it];
    }
    __syncthreads();
    if (k0 + GT_KC < bw) fetch(k0 + GT_KC);
#pragma unroll
    for (int kk = 0; kk < GT_KC; kk += 16) {
      uint32_t af[3][4];
#pragma unroll
      for (int q = 0; q < 3; ++q) {
        const __nv_bfloat16* base = &As[q][warp * 16 + gq][kk + cq * 2];
        af[q][0] = *reinterpret_cast<const uint32_t*>(base);
        af[q][1] = *reinterpret_cast<const uint32_t*>(base + 8 * GT_LD);
        af[q][2] = *reinterpret_cast<const uint32_t*>(base + 8);
        af[q][3] = *reinterpret_cast<const uint32_t*>(base + 8 * GT_LD + 8);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const __nv_bfloat16* wb = &Ws[j * 8 + gq][kk + cq * 2];
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(wb), b1 = *reinterpret_cast<const uint32_t*>(wb + 8);
        mma_bf16_16816(acc[j], af[2], b0, b1);      // the smallest terms first
        mma_bf16_16816(acc[j], af[1], b0, b1);
        mma_bf16_16816(acc[j], af[0], b0, b1);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int n = n0 + (j % 4) * 8 + cq * 2;
    float* dst = gates + (j < 4 ? 0 : W) + (size_t)blk * bw + n;
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
      const int t = t0 + warp * 16 + gq + hrow * 8;
      if (t < n_tokens) {
        if (n < bw) dst[(size_t)t * ldg] = acc[j][hrow * 2];
        if (n + 1 < bw) dst[(size_t)t * ldg + 1] = acc[j][hrow * 2 + 1];
      }
    }
  }
}

// mid = g sigmoid(alpha g) (v + 1) with g = min(gate, limit), v = clamp(up, -limit, limit); gu [tokens][2 F] float32 = gate | up
template <typename TO>
__global__ void clamped_glu_kernel(const float* __restrict__ gu, TO* __restrict__ mid, int F, float limit, float alpha, float shift,
                                   const float* __restrict__ bias, float* __restrict__ x, const float* __restrict__ x_bias, int D) {
  pdl_launch_dependents();
  pdl_wait();
  if (x != nullptr)      // the bias of the projection that follows, added to the rows that its residual epilogue adds to
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < D; i += gridDim.y * blockDim.x) x[(size_t)blockIdx.x * D + i] += x_bias[i];
  const float* row = gu + (size_t)blockIdx.x * 2 * F;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < F; i += gridDim.y * blockDim.x) {    // (few tokens: several blocks a token)
    float g = row[i] + (bias ? bias[i] : 0.f), v = row[F + i] + (bias ? bias[F + i] : 0.f);
    if (limit > 0.f) {
      g = fminf(g, limit);
      v = fminf(fmaxf(v, -limit), limit);
    }
    mid[(size_t)blockIdx.x * F + i] = from_f32<TO>(g * sigmoid_f(alpha * g) * (v + shift));
  }
}

}  // namespace edgelm

using namespace edgelm;

// gates [tokens][>= 2 W] (r | i pre-activations, row pitch ldg), u [tokens][W..] (pitch ldu), y [tokens][W..] (pitch ldy);
// `single`: every sequence brings one token (token t is sequence t).  Otherwise `tok_seq` [tokens] names every token's
// sequence, `scratch` holds 2 * segments * W floats, segments = ceil(tokens / RG_SEG), and `gates` is overwritten (decays | inputs).
extern "C" int edgelm_rglru_scan(float* gates, int ldg, const float* br, const float* bi, const float* u, int ldu, const float* c,
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
    float* seg = scratch;
    const dim3 grid((W + 31) / 32, segs), block(RG_WARPS * 32);
    launch_pdl(bit, rglru_compose_kernel, grid, block, (size_t)0, stream, gates, ldg, br, bi, u, ldu, c, (const float*)state, seg, seq_tok0, seq_slot, tok_seq, n_tokens, W);
    if (out_dtype == DT_F32) launch_pdl(bit, rglru_walk_kernel<float>, grid, block, (size_t)0, stream, (const float*)gates, ldg, y, ldy, by, (const float*)seg, state, (float*)out, seq_tok0, seq_slot, tok_seq, n_tokens, W);
    else launch_pdl(bit, rglru_walk_kernel<__nv_bfloat16>, grid, block, (size_t)0, stream, (const float*)gates, ldg, y, ldy, by, (const float*)seg, state, (__nv_bfloat16*)out, seq_tok0, seq_slot, tok_seq, n_tokens, W);
  }
  EL_LAUNCH_CHECK("rglru_scan");
  return 0;
}

// gates [tokens][>= 2 W] float32 <- the block-diagonal products of u [tokens][W..] float32 with ra and ri [blocks][bw][bw] bfloat16
extern "C" int edgelm_rglru_gates(const float* u, int ldu, const void* w_ra, const void* w_ri, float* gates, int ldg, int n_tokens, int W,
                                  int blocks, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && W > 0 && blocks > 0 && W % blocks == 0 && ldu >= W && ldg >= 2 * W && blocks <= 65535, "rglru_gates: bad sizes (width %d, %d blocks)", W, blocks);
  const int bw = W / blocks;
  const dim3 grid((n_tokens + GT_M - 1) / GT_M, (bw + GT_N - 1) / GT_N, blocks), block(128);
  launch_pdl(pdl_bit_for_tokens(n_tokens), rglru_gates_mma_kernel, grid, block, (size_t)0, stream, u, ldu, (const __nv_bfloat16*)w_ra,
             (const __nv_bfloat16*)w_ri, gates, ldg, n_tokens, W, bw);
  EL_LAUNCH_CHECK("rglru_gates");
  return 0;
}

// mid = g sigmoid(alpha g) (v + shift) with g = gate + bias, v = up + bias, both clamped (g from above, v on both sides) when
// limit > 0; `bias` [2 F] may be null.  limit 0, alpha 1, shift 0: SwiGLU.
// `x` [tokens][D] with `x_bias` [D] (or null): x[t] += x_bias as well, in the same launch.
extern "C" int edgelm_clamped_glu(const float* gu, void* mid, int out_dtype, int n_tokens, int F, float limit, float alpha, float shift,
                                  const float* bias, float* x, const float* x_bias, int D, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && F > 0 && limit >= 0.f, "clamped_glu: bad sizes");
  // a token's row is a chain of trips to memory when one block walks it: with few tokens a block takes 256 or 512 channels
  const int per_block = F >= 1024 ? 512 : 256;
  const dim3 grid(n_tokens, n_tokens <= 64 ? (F + per_block - 1) / per_block : 1), block(F >= 1024 ? 256 : 128);
  const int bit = pdl_bit_for_tokens(n_tokens);
  if (out_dtype == DT_F32) launch_pdl(bit, clamped_glu_kernel<float>, grid, block, (size_t)0, stream, gu, (float*)mid, F, limit, alpha, shift, bias, x, x_bias, D);
  else if (out_dtype == DT_BF16) launch_pdl(bit, clamped_glu_kernel<__nv_bfloat16>, grid, block, (size_t)0, stream, gu, (__nv_bfloat16*)mid, F, limit, alpha, shift, bias, x, x_bias, D);
  else EL_REFUSE(false, "clamped_glu: unknown dtype code %d", out_dtype);
  EL_LAUNCH_CHECK("clamped_glu");
  return 0;
}
