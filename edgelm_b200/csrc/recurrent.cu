// Kernels of mixers that carry a fixed-size state from token to token: the blend of a token with the one
// before it (token shift), a short causal convolution over channels, the selective state-space recurrence
// (state N x P per head, scalar decay per head and token), the decayed outer-product recurrence with a bonus
// for the current token (state K x V per head, decay per key channel and token), the decay's low-rank
// projection, and the gated group RMS norm that follows both recurrences.
//
// Tokens of all sequences are packed along the first axis; `seq_tok0[s] .. seq_tok0[s + 1] - 1` are the packed
// rows of the batch's sequence s, `seq_slot[s]` the row of its state.  States, decays, step sizes, norms and the
// recurrences themselves are float32 in both precisions; `T*` names the storage type of activations that feed a
// matrix product (float or bfloat16).
#include "common.cuh"

namespace edgelm {

__device__ __forceinline__ float silu_exact(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_exact(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.f); }

// ------------------------------------------------------------------ blend with the previous token
// out[m][t][:] = a + (prev - a) * mu[m][:], a = in[t], prev = in[t - 1], or the state row for the first token
// that a sequence brings to this step (zeros at a sequence's start).  With `move_state` the block of that first token,
// the only one that reads the sequence's state row, then writes the sequence's last row of this step into it (each
// thread the elements it has just read), so that the state needs no kernel of its own.
template <typename TIn, typename TOut>
__global__ void shift_mix_kernel(const TIn* __restrict__ in, const float* state, const float* __restrict__ mu,
                                 TOut* __restrict__ out, const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ seq_tok0,
                                 const int32_t* __restrict__ seq_slot, int n_tokens, int dim, int n_mix, int move_state) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  const int t = blockIdx.x;
  const int s = tok_seq[t];
  const bool first = t == seq_tok0[s];
  float* st = const_cast<float*>(state) + (size_t)seq_slot[s] * dim;
  const TIn* cur = in + (size_t)t * dim;
  const TIn* last = in + (size_t)(seq_tok0[s + 1] - 1) * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float a = to_f32(cur[i]);
    const float p = first ? st[i] : to_f32(cur[i - dim]);
    const float d = p - a;
    for (int m = 0; m < n_mix; ++m) out[((size_t)m * n_tokens + t) * dim + i] = from_f32<TOut>(a + d * mu[(size_t)m * dim + i]);
    if (first && move_state) st[i] = to_f32(last[i]);
  }
}

// state[slot(s)][:] = in[last row of s][:]
template <typename TIn>
__global__ void save_last_rows_kernel(const TIn* __restrict__ in, float* __restrict__ state, const int32_t* __restrict__ seq_tok0,
                                      const int32_t* __restrict__ seq_slot, int dim) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  const int s = blockIdx.x;
  const int t = seq_tok0[s + 1] - 1;
  float* st = state + (size_t)seq_slot[s] * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) st[i] = to_f32(in[(size_t)t * dim + i]);
}

// ------------------------------------------------------------------ short causal convolution + silu
// Channel c of token t: silu(b[c] + sum_j w[c][j] * in[t - (taps - 1) + j][c]); inputs before the step come from
// the state [slot][taps - 1][C] (oldest first; zeros before a sequence's start).  `u` holds the inputs at column
// `off + c` of rows of `ldu` floats.  `in_bias` (optional): added to every input that `u` brings, before the
// convolution (a projection's bias; the state keeps inputs with it, and the zeros before a sequence's start stay zeros).
// `b` may be null (no bias on the result); `act` 0: no activation.  `move_state` (steps of one token a sequence only: the
// thread of (token, channel) is then the only one that touches the sequence's tail of that channel): the tail moves on
// by the token's input here, and no second launch is needed.
__global__ void conv_silu_kernel(const float* __restrict__ u, int ldu, int off, const float* __restrict__ w,
                                 const float* __restrict__ b, float* state, float* __restrict__ out,
                                 const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ seq_tok0,
                                 const int32_t* __restrict__ seq_slot, int C, int taps, const float* __restrict__ in_bias, int act,
                                 int move_state) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  const int t = blockIdx.x;
  const int s = tok_seq[t];
  const int t0 = seq_tok0[s];
  const int k = t - t0;
  float* st = state + (size_t)seq_slot[s] * (taps - 1) * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {   // (few tokens: several blocks a token)
    float acc = b ? b[c] : 0.f;
    const float ib = in_bias ? in_bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int r = k - (taps - 1) + j;
      const float v = r >= 0 ? u[(size_t)(t0 + r) * ldu + off + c] + ib : st[(size_t)(taps - 1 + r) * C + c];
      acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    out[(size_t)t * C + c] = act ? silu_exact(acc) : acc;
    if (move_state) {      // (k == 0: every row of the tail was read above; row j takes row j + 1, the last one the token's input)
      for (int j = 0; j + 2 < taps; ++j) st[(size_t)j * C + c] = st[(size_t)(j + 1) * C + c];
      st[(size_t)(taps - 2) * C + c] = u[(size_t)t * ldu + off + c] + ib;
    }
  }
}

// The state after the step: the last taps - 1 inputs of each sequence.  A thread owns a channel and walks the
// rows upwards, so that a row it still has to read (one further on) is never overwritten before.
__global__ void conv_state_update_kernel(const float* __restrict__ u, int ldu, int off, float* __restrict__ state,
                                         const int32_t* __restrict__ seq_tok0, const int32_t* __restrict__ seq_slot, int C, int taps,
                                         const float* __restrict__ in_bias) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  const int s = blockIdx.x;
  const int t0 = seq_tok0[s], n = seq_tok0[s + 1] - t0;
  float* st = state + (size_t)seq_slot[s] * (taps - 1) * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    const float ib = in_bias ? in_bias[c] : 0.f;
    for (int j = 0; j < taps - 1; ++j) {
      const int r = n - (taps - 1) + j;
      st[(size_t)j * C + c] = r >= 0 ? u[(size_t)(t0 + r) * ldu + off + c] + ib : st[(size_t)(j + n) * C + c];
    }
  }
}

// Sums over the warp of U values a lane at once: at each of the first log2(U) steps a lane keeps one half of its values
// and hands the other half to its partner, so U values cost U - 1 + log2(32 / U) shuffles instead of 5 U.  Afterwards the
// sum of value i is held by the lanes [i * 32 / U, (i + 1) * 32 / U).
template <int U>
__device__ __forceinline__ float warp_sums(float (&acc)[U], int lane) {
  int off = 16;
#pragma unroll
  for (int n = U; n > 1; n >>= 1) {
    const int half = n >> 1;
    const bool hi = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float keep = hi ? acc[i + half] : acc[i], send = hi ? acc[i] : acc[i + half];
      acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
    off >>= 1;
  }
  float v = acc[0];
  for (; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// dt = softplus(raw + bias) and the decay exp(-exp(A_log) dt) of every (token, head), once for all the warps of a head:
// dta[t][h] = dt, dta[t][H + h] = decay.
__global__ void ssm_steps_kernel(const float* __restrict__ u, int ldu, int dt_off, const float* __restrict__ dt_bias,
                                 const float* __restrict__ A_log, float* __restrict__ dta, int n_tokens, int H) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * H) return;
  const int t = i / H, h = i - t * H;
  const float dt = softplus_exact(u[(size_t)t * ldu + dt_off + h] + dt_bias[h]);
  dta[(size_t)t * 2 * H + h] = dt;
  dta[(size_t)t * 2 * H + H + h] = expf(-expf(A_log[h]) * dt);
}

// ------------------------------------------------------------------ selective state-space recurrence
// Per head h (group g = h / (H / G)) and token t, with dt = softplus(dt_raw + dt_bias[h]) and a = exp(-exp(A_log[h]) dt):
//   S <- a S + dt B_t x_t^T      (S is N x P)
//   y_t = S^T C_t + D[h] x_t
// A warp owns one column p of one head of one sequence; lane l holds the rows n = l NK .. l NK + NK - 1 in registers, so
// a token costs a handful of multiply-adds and a share of a warp sum, and nothing is exchanged between warps.  The step
// sizes and decays come from `ssm_steps_kernel`.
// (The outer-product recurrence further down takes its tokens U at a time through registers: their inputs are requested
// together, one set ahead of the set that is being computed, and the warp sums of a set are done together.)
constexpr int SCAN_WARPS = 8;

__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_LEFT> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_LEFT) : "memory"); }

constexpr int SCAN_CHUNK = 8;     // tokens a stage of the ring holds
constexpr int SCAN_MAX_STAGES = 4;

// The block's eight warps (eight columns p of one head) need the same B_t, C_t, step size and decay, and one x each:
// all threads bring SCAN_CHUNK tokens' worth of these into a ring in shared memory with asynchronous copies, `stages`
// - 1 chunks ahead of the chunk that is being computed, so that a token's inputs are on the chip long before its turn
// and are fetched once a block, not once a warp.  A token's slot: B [NP], C [NP], x [SCAN_WARPS], dt, decay, (pad).
template <int NK, bool EXACT>     // EXACT: N == 32 NK, every lane's rows exist
__global__ void __launch_bounds__(SCAN_WARPS * 32)
ssm_scan_kernel(const float* __restrict__ xbc, int C, int inner, int G, int N, const float* __restrict__ u, int ldu,
                const float* __restrict__ dta, const float* __restrict__ Dp,
                float* __restrict__ state, float* __restrict__ y, const int32_t* __restrict__ seq_tok0,
                const int32_t* __restrict__ seq_slot, int H, int P, float* __restrict__ conv_state, int conv_off, int taps, int vec,
                int stages) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  extern __shared__ __align__(16) float ring[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = blockIdx.x / H, h = blockIdx.x - s * H;
  if (conv_state != nullptr && taps > 1 && h == 0 && blockIdx.y == 0) {
    // the convolution that fed this kernel has read its tail; one block a sequence moves the tail on to the step's last
    // inputs (a thread a channel, rows upwards: a row still to be read lies further on than the row being written)
    const int c0 = seq_tok0[s], n = seq_tok0[s + 1] - c0;
    float* cs = conv_state + (size_t)seq_slot[s] * (taps - 1) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x)
      for (int j = 0; j < taps - 1; ++j) {
        const int r = n - (taps - 1) + j;
        cs[(size_t)j * C + c] = r >= 0 ? u[(size_t)(c0 + r) * ldu + conv_off + c] : cs[(size_t)(j + n) * C + c];
      }
  }
  const int p0 = blockIdx.y * SCAN_WARPS, p = p0 + warp;
  const bool active = p < P;
  const int g = h / (H / G);
  const int t0 = seq_tok0[s], t1 = seq_tok0[s + 1];
  const int NP = (N + 3) & ~3, slot = 2 * NP + SCAN_WARPS + 4;
  const int n0 = lane * NK;            // this lane's rows: n0 .. n0 + NK - 1
  float* sp = state + (((size_t)seq_slot[s] * H + h) * P + (active ? p : 0)) * N;
  float S[NK];
#pragma unroll
  for (int k = 0; k < NK; ++k) S[k] = active && n0 + k < N ? sp[n0 + k] : 0.f;
  const float Dh = Dp[h];
  const int xo = h * P + p0, bo = inner + g * N, co = inner + G * N + g * N;
  const int n_chunks = (t1 - t0 + SCAN_CHUNK - 1) / SCAN_CHUNK;

  // which copies this thread makes in every chunk: worked out once (no division inside the loop)
  const int per_tok = vec ? 2 * (NP >> 2) : 2 * N;           // copies of B and C a token
  const int step_i = blockDim.x / per_tok, step_r = blockDim.x - step_i * per_tok;
  const int first_i = threadIdx.x / per_tok, first_r = threadIdx.x - first_i * per_tok;
  const int small_i = threadIdx.x / (SCAN_WARPS + 2), small_r = threadIdx.x - small_i * (SCAN_WARPS + 2);   // x, dt, decay
  const float* small_src = small_r < SCAN_WARPS ? xbc + xo + min(small_r, P - 1 - p0) : dta + (size_t)(small_r - SCAN_WARPS) * H + h;
  const size_t small_ld = small_r < SCAN_WARPS ? (size_t)C : (size_t)2 * H;
  auto issue = [&](int chunk, int stage) {   // the copies of one chunk into its stage (tokens past the end repeat the last one)
    if (chunk < n_chunks) {
      float* base = ring + (size_t)stage * SCAN_CHUNK * slot;
      const int tc = t0 + chunk * SCAN_CHUNK;
      for (int i = first_i, r = first_r; i < SCAN_CHUNK;) {
        const float* row = xbc + (size_t)min(tc + i, t1 - 1) * C;
        float* dst = base + (size_t)i * slot;
        if (vec) {
          const int half = NP >> 2, which = r >= half, q = (r - (which ? half : 0)) << 2;
          cp_async_16(dst + (which ? NP : 0) + q, row + (which ? co : bo) + q);
        } else {
          const int which = r >= N, q = r - (which ? N : 0);
          cp_async_4(dst + (which ? NP : 0) + q, row + (which ? co : bo) + q);
        }
        i += step_i;
        r += step_r;
        if (r >= per_tok) { r -= per_tok; ++i; }
      }
      if (small_i < SCAN_CHUNK)
        cp_async_4(base + (size_t)small_i * slot + 2 * NP + small_r, small_src + (size_t)min(tc + small_i, t1 - 1) * small_ld);
    }
    cp_async_commit();                 // (an empty group keeps the count of groups in step with the chunks)
  };

  for (int c = 0; c < stages - 1; ++c) issue(c, c);
  int stage = 0;                       // the stage of the chunk being computed; the one before it is refilled
  for (int chunk = 0; chunk < n_chunks; ++chunk) {
    // all but the newest stages - 2 groups are complete: chunk `chunk` has landed
    if (stages == 4) cp_async_wait<2>(); else if (stages == 3) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();                   // everybody's copies of this chunk are visible; everybody is done with chunk - 1
    issue(chunk + stages - 1, stage == 0 ? stages - 1 : stage - 1);         // into the stage that chunk - 1 used
    const float* base = ring + (size_t)stage * SCAN_CHUNK * slot;
    stage = stage + 1 == stages ? 0 : stage + 1;
    const int tb = t0 + chunk * SCAN_CHUNK;
    float acc[SCAN_CHUNK], xs[SCAN_CHUNK];
    auto token = [&](int i, const float* tok) {
      const float a = tok[2 * NP + SCAN_WARPS + 1], dx = tok[2 * NP + SCAN_WARPS] * xs[i];
      float Bn[NK], Cn[NK];
      if (NK >= 4) {
#pragma unroll
        for (int k = 0; k < NK; k += 4) {
          const bool in = EXACT || n0 + k < N;
          const float4 b4 = in ? *reinterpret_cast<const float4*>(tok + n0 + k) : make_float4(0.f, 0.f, 0.f, 0.f);
          const float4 c4 = in ? *reinterpret_cast<const float4*>(tok + NP + n0 + k) : make_float4(0.f, 0.f, 0.f, 0.f);
          Bn[k] = b4.x; Bn[k + 1] = b4.y; Bn[k + 2] = b4.z; Bn[k + 3] = b4.w;
          Cn[k] = c4.x; Cn[k + 1] = c4.y; Cn[k + 2] = c4.z; Cn[k + 3] = c4.w;
        }
      } else if (NK == 2 && EXACT) {
        const float2 b2 = *reinterpret_cast<const float2*>(tok + n0), c2 = *reinterpret_cast<const float2*>(tok + NP + n0);
        Bn[0] = b2.x; Bn[1] = b2.y; Cn[0] = c2.x; Cn[1] = c2.y;
      } else {
#pragma unroll
        for (int k = 0; k < NK; ++k) {
          Bn[k] = EXACT || n0 + k < N ? tok[n0 + k] : 0.f;
          Cn[k] = EXACT || n0 + k < N ? tok[NP + n0 + k] : 0.f;
        }
      }
#pragma unroll
      for (int k = 0; k < NK; ++k) {
        const bool in = EXACT || n0 + k < N;    // (a vector piece may reach past N into the slot's padding)
        S[k] = in ? fmaf(a, S[k], dx * Bn[k]) : 0.f;
        acc[i] = in ? fmaf(S[k], Cn[k], acc[i]) : acc[i];
      }
    };
    const float* tok = base;
    if (tb + SCAN_CHUNK <= t1) {       // a whole chunk: no token needs a check
#pragma unroll
      for (int i = 0; i < SCAN_CHUNK; ++i, tok += slot) {
        acc[i] = 0.f;
        xs[i] = tok[2 * NP + warp];
        token(i, tok);
      }
    } else {
#pragma unroll
      for (int i = 0; i < SCAN_CHUNK; ++i, tok += slot) {
        acc[i] = 0.f;
        xs[i] = tok[2 * NP + warp];
        if (tb + i < t1) token(i, tok);
      }
    }
    const float sum = warp_sums<SCAN_CHUNK>(acc, lane);
    const int i = lane / (32 / SCAN_CHUNK);
    if (active && (lane & (32 / SCAN_CHUNK - 1)) == 0 && tb + i < t1) {
      float xi = xs[0];
#pragma unroll
      for (int q = 1; q < SCAN_CHUNK; ++q) xi = i == q ? xs[q] : xi;
      y[(size_t)(tb + i) * inner + xo + warp] = sum + Dh * xi;
    }
  }
  cp_async_wait<0>();
  if (active) {
#pragma unroll
    for (int k = 0; k < NK; ++k)
      if (n0 + k < N) sp[n0 + k] = S[k];
  }
}

// ------------------------------------------------------------------ decayed outer-product recurrence with a bonus
// Per head, key channel i and value channel j:
//   o_t[j] = sum_i (S[i][j] + bonus[i] k_t[i] v_t[j]) r_t[i]
//   S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j]
// A warp owns one value channel j; lane l holds the key channels i = l, l + 32, ...  r, k, v, w: [tokens][H * K]
// (value size = key size K); state [slot][H][K (j)][K (i)].
template <int NK, int U>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
wkv_scan_kernel(const float* __restrict__ r, const float* __restrict__ kk, const float* __restrict__ v, const float* __restrict__ w,
                const float* __restrict__ bonus, float* __restrict__ state, float* __restrict__ o,
                const int32_t* __restrict__ seq_tok0, const int32_t* __restrict__ seq_slot, int H, int K) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = blockIdx.x / H, h = blockIdx.x - s * H;
  const int j = blockIdx.y * (blockDim.x >> 5) + warp;
  if (j >= K) return;
  const int t0 = seq_tok0[s], t1 = seq_tok0[s + 1];
  float* sp = state + (((size_t)seq_slot[s] * H + h) * K + j) * K;
  float S[NK], bn[NK];
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const int i = lane + 32 * k;
    S[k] = i < K ? sp[i] : 0.f;
    bn[k] = i < K ? bonus[h * K + i] : 0.f;
  }
  const int ld = H * K, ho = h * K;
  struct Inputs { float vj[U], rr[U][NK], kv[U][NK], ww[U][NK]; };
  auto load = [&](int tb, Inputs& in) {
#pragma unroll
    for (int q = 0; q < U; ++q) {
      const size_t row = (size_t)min(tb + q, t1 - 1) * ld + ho;
      in.vj[q] = v[row + j];
#pragma unroll
      for (int k = 0; k < NK; ++k) {
        const int i = lane + 32 * k;
        in.rr[q][k] = i < K ? r[row + i] : 0.f;
        in.kv[q][k] = i < K ? kk[row + i] : 0.f;
        in.ww[q][k] = i < K ? w[row + i] : 0.f;
      }
    }
  };
  auto compute = [&](int tb, const Inputs& in) {
    float acc[U];
#pragma unroll
    for (int q = 0; q < U; ++q) {
      acc[q] = 0.f;
      if (tb + q < t1) {
#pragma unroll
        for (int k = 0; k < NK; ++k) {
          const float x = in.kv[q][k] * in.vj[q];
          acc[q] = fmaf(fmaf(bn[k], x, S[k]), in.rr[q][k], acc[q]);
          S[k] = fmaf(in.ww[q][k], S[k], x);
        }
      }
    }
    const float sum = warp_sums<U>(acc, lane);
    const int q = lane / (32 / U);
    if ((lane & (32 / U - 1)) == 0 && tb + q < t1) o[(size_t)(tb + q) * ld + ho + j] = sum;
  };
  Inputs ia, ib;
  if (t0 < t1) load(t0, ia);
  for (int tb = t0; tb < t1; tb += 2 * U) {
    if (tb + U < t1) load(tb + U, ib);
    compute(tb, ia);
    if (tb + U < t1) {
      if (tb + 2 * U < t1) load(tb + 2 * U, ia);
      compute(tb + U, ib);
    }
  }
#pragma unroll
  for (int k = 0; k < NK; ++k)
    if (lane + 32 * k < K) sp[lane + 32 * k] = S[k];
}

// ------------------------------------------------------------------ the decay from its low-rank projection
// out[t][c] = exp(-exp(w0[c] + sum_l W2[c][l] tanh(a[t][l]))), all in float32 (W2 in its storage type).
template <typename TW>
__global__ void lowrank_decay_kernel(const float* __restrict__ a, const TW* __restrict__ w2, const float* __restrict__ w0,
                                     float* __restrict__ out, int C, int L) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  extern __shared__ float th[];
  const int t = blockIdx.x;
  for (int l = threadIdx.x; l < L; l += blockDim.x) th[l] = tanhf(a[(size_t)t * L + l]);
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = w0[c];
    const TW* row = w2 + (size_t)c * L;
    for (int l = 0; l < L; ++l) acc = fmaf(to_f32(row[l]), th[l], acc);
    out[(size_t)t * C + c] = expf(-expf(acc));
  }
}

// ------------------------------------------------------------------ gated RMS norm in equal groups
// A row of `inner` values in `groups` equal parts, each divided by its own root mean square.
//   gate_first:  v = y * act(gate); out = v / rms(v) * w
//   else:        out = y / rms(y) * w * act(gate)
// act = silu, or with `gate_sigmoid` the sigmoid itself.
template <typename TOut>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ gate, int ldg,
                                        const float* __restrict__ w, TOut* __restrict__ out, int inner, int groups, float eps,
                                        int gate_first, int gate_sigmoid) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  __shared__ float red[33];
  const int t = blockIdx.x, g = blockIdx.y, gs = inner / groups;
  const float* yr = y + (size_t)t * inner + (size_t)g * gs;
  const float* gr = gate + (size_t)t * ldg + (size_t)g * gs;
  const float* wr = w + (size_t)g * gs;
  float ss = 0.f;
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float v = gate_first ? yr[i] * (gate_sigmoid ? 1.0f / (1.0f + expf(-gr[i])) : silu_exact(gr[i])) : yr[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
  TOut* orow = out + (size_t)t * inner + (size_t)g * gs;
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float sg = gate_sigmoid ? 1.0f / (1.0f + expf(-gr[i])) : silu_exact(gr[i]);
    orow[i] = from_f32<TOut>(gate_first ? yr[i] * sg * inv * wr[i] : yr[i] * inv * wr[i] * sg);
  }
}

// ------------------------------------------------------------------ x += rmsnorm(a y1 + b y2) * w  (+ a copy of x in the compute type)
template <typename TCast>
__global__ void rmsnorm_add_kernel(float* __restrict__ x, const float* __restrict__ y1, float a, const float* __restrict__ y2, float b,
                                   const float* __restrict__ w, TCast* __restrict__ xc, int dim, float eps) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* r1 = y1 + (size_t)t * dim;
  const float* r2 = y2 ? y2 + (size_t)t * dim : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = r2 ? a * r1[i] + b * r2[i] : a * r1[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  float* xr = x + (size_t)t * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = r2 ? a * r1[i] + b * r2[i] : a * r1[i];
    const float nx = xr[i] + v * inv * w[i];
    xr[i] = nx;
    if (xc) xc[(size_t)t * dim + i] = from_f32<TCast>(nx);
  }
}

// out = a y1 + b y2, or with `add` out += a y1 + b y2
__global__ void scaled_sum_kernel(const float* __restrict__ y1, float a, const float* __restrict__ y2, float b, float* __restrict__ out, size_t n, int add) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = a * y1[i] + b * y2[i];
    out[i] = add ? out[i] + v : v;
  }
}

}  // namespace edgelm

using namespace edgelm;

extern "C" int edgelm_scaled_sum(const float* y1, float a, const float* y2, float b, float* out, long long n, int add, cudaStream_t stream) {
  if (n == 0) return 0;
  EL_REFUSE(n > 0, "scaled_sum: bad size");
  const long long blocks = (n + 255) / 256;
  scaled_sum_kernel<<<(unsigned)(blocks < 4096 ? blocks : 4096), 256, 0, stream>>>(y1, a, y2, b, out, (size_t)n, add);
  EL_LAUNCH_CHECK("scaled_sum");
  return 0;
}

static inline int row_threads(int dim) { return dim >= 1024 ? 256 : 128; }

extern "C" int edgelm_shift_mix(const void* in, int in_dtype, float* state, const float* mu, void* out, int out_dtype,
                                const int32_t* tok_seq, const int32_t* seq_tok0, const int32_t* seq_slot, int n_tokens, int dim,
                                int n_mix, int move_state, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && dim > 0 && n_mix > 0, "shift_mix: bad sizes tokens=%d dim=%d mixes=%d", n_tokens, dim, n_mix);
  const dim3 grid(n_tokens), block(row_threads(dim));
#define EL_SM(TI, TO) launch_pdl(pdl_bit_for_tokens(n_tokens), shift_mix_kernel<TI, TO>, dim3(grid), dim3(block), (size_t)(0), stream, (const TI*)in, state, mu, (TO*)out, tok_seq, seq_tok0, seq_slot, n_tokens, dim, n_mix, move_state)
  if (in_dtype == DT_F32 && out_dtype == DT_F32) EL_SM(float, float);
  else if (in_dtype == DT_F32 && out_dtype == DT_BF16) EL_SM(float, __nv_bfloat16);
  else if (in_dtype == DT_BF16 && out_dtype == DT_BF16) EL_SM(__nv_bfloat16, __nv_bfloat16);
  else EL_REFUSE(false, "shift_mix: dtype codes %d -> %d are not taken", in_dtype, out_dtype);
#undef EL_SM
  EL_LAUNCH_CHECK("shift_mix");
  return 0;
}

extern "C" int edgelm_save_last_rows(const void* in, int in_dtype, float* state, const int32_t* seq_tok0, const int32_t* seq_slot,
                                     int n_seqs, int dim, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  EL_REFUSE(n_seqs > 0 && dim > 0, "save_last_rows: bad sizes");
  const int n_tokens = n_seqs;   // (as many launches' worth of blocks as a decode step has tokens)
  if (in_dtype == DT_F32) launch_pdl(pdl_bit_for_tokens(n_tokens), save_last_rows_kernel<float>, dim3(n_seqs), dim3(row_threads(dim)), (size_t)(0), stream, (const float*)in, state, seq_tok0, seq_slot, dim);
  else if (in_dtype == DT_BF16) launch_pdl(pdl_bit_for_tokens(n_tokens), save_last_rows_kernel<__nv_bfloat16>, dim3(n_seqs), dim3(row_threads(dim)), (size_t)(0), stream, (const __nv_bfloat16*)in, state, seq_tok0, seq_slot, dim);
  else EL_REFUSE(false, "save_last_rows: unknown dtype code %d", in_dtype);
  EL_LAUNCH_CHECK("save_last_rows");
  return 0;
}

// The convolution over the step's tokens and, with `update_state`, the state for the next step after it (a second launch).
extern "C" int edgelm_conv_act(const float* u, int ldu, int off, const float* w, const float* b, float* state, float* out,
                               const int32_t* tok_seq, const int32_t* seq_tok0, const int32_t* seq_slot, int n_tokens, int n_seqs,
                               int C, int taps, int update_state, const float* in_bias, int act, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && n_seqs > 0 && C > 0 && taps >= 1 && off >= 0 && off + C <= ldu, "conv_silu: bad sizes C=%d taps=%d", C, taps);
  // several blocks a token, so that a thread's loads are few and many blocks overlap theirs: 4 channels a thread in steps of
  // few tokens, 2 in prompt steps (one block a token there left a thread ten channels in a row at a width of 2,560)
  const int per_thread = n_tokens >= 256 ? 2 : 4;
  const int col_blocks = (C + per_thread * row_threads(C) - 1) / (per_thread * row_threads(C));
  // a step of one token a sequence (as many tokens as sequences) moves the tail on in the same launch
  const int fused_tail = taps > 1 && update_state && n_tokens == n_seqs;
  launch_pdl(pdl_bit_for_tokens(n_tokens), conv_silu_kernel, dim3(n_tokens, col_blocks), dim3(row_threads(C)), (size_t)(0), stream, u, ldu, off, w, b, state, out, tok_seq, seq_tok0, seq_slot, C, taps, in_bias, act, fused_tail);
  EL_LAUNCH_CHECK("conv_silu");
  if (taps > 1 && update_state && !fused_tail) {
    launch_pdl(pdl_bit_for_tokens(n_tokens), conv_state_update_kernel, dim3(dim3(n_seqs, (C + 255) / 256)), dim3(256), (size_t)(0), stream, u, ldu, off, state, seq_tok0, seq_slot, C, taps, in_bias);
    EL_LAUNCH_CHECK("conv_state_update");
  }
  return 0;
}

// The tails after a step, by themselves: for a caller whose own kernel ran the filter (and read the old tails) already.
extern "C" int edgelm_conv_tail_update(const float* u, int ldu, int off, float* state, const int32_t* seq_tok0, const int32_t* seq_slot,
                                       int n_seqs, int C, int taps, const float* in_bias, cudaStream_t stream) {
  if (n_seqs == 0 || taps <= 1) return 0;
  EL_REFUSE(n_seqs > 0 && C > 0 && ldu >= off + C, "conv_tail_update: bad sizes");
  const dim3 grid(n_seqs, (C + 255) / 256), block(256);
  launch_pdl(pdl_bit_for_tokens(n_seqs), conv_state_update_kernel, grid, block, (size_t)0, stream, u, ldu, off, state, seq_tok0, seq_slot, C, taps, in_bias);
  EL_LAUNCH_CHECK("conv_tail_update");
  return 0;
}

extern "C" int edgelm_conv_silu(const float* u, int ldu, int off, const float* w, const float* b, float* state, float* out,
                                const int32_t* tok_seq, const int32_t* seq_tok0, const int32_t* seq_slot, int n_tokens, int n_seqs,
                                int C, int taps, int update_state, cudaStream_t stream) {
  return edgelm_conv_act(u, ldu, off, w, b, state, out, tok_seq, seq_tok0, seq_slot, n_tokens, n_seqs, C, taps, update_state, nullptr, 1, stream);
}

// `conv_state` (may be null): the tail [slot][taps - 1][C] of the convolution whose inputs lie at u[:, conv_off + c];
// the kernel then moves it on to the step's last inputs (`edgelm_conv_silu` with `update_state` 0 left that to it).
// `dta`: scratch of 2 * n_tokens * H floats for the step sizes and decays (a launch of its own fills it).
extern "C" int edgelm_ssm_scan(const float* xbc, int C, int inner, int G, int N, const float* u, int ldu, int dt_off,
                               const float* dt_bias, const float* A_log, const float* Dp, float* state, float* y,
                               const int32_t* seq_tok0, const int32_t* seq_slot, int n_seqs, int H, int P, float* conv_state,
                               int conv_off, int taps, float* dta, int n_tokens, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  EL_REFUSE(n_seqs > 0 && H > 0 && P > 0 && G > 0 && H % G == 0 && inner == H * P && C == inner + 2 * G * N,
            "ssm_scan: sizes do not fit (heads %d, groups %d, head size %d, inner %d, channels %d)", H, G, P, inner, C);
  EL_REFUSE(N >= 1 && N <= 256, "ssm_scan: a state of %d rows per head is not taken (1 to 256)", N);
  EL_REFUSE(dta != nullptr && n_tokens > 0, "ssm_scan: needs room for the step sizes and decays of %d tokens", n_tokens);
  launch_pdl(pdl_bit_for_tokens(n_tokens), ssm_steps_kernel, dim3((n_tokens * H + 255) / 256), dim3(256), (size_t)(0), stream, u, ldu, dt_off, dt_bias, A_log, dta, n_tokens, H);
  EL_LAUNCH_CHECK("ssm_steps");
  const dim3 grid(n_seqs * H, (P + SCAN_WARPS - 1) / SCAN_WARPS), block(SCAN_WARPS * 32);
  // B and C rows as 16-byte pieces where every row starts on such a boundary
  const int vec = (uintptr_t)xbc % 16 == 0 && C % 4 == 0 && inner % 4 == 0 && N % 4 == 0;
  const int slot = 2 * ((N + 3) & ~3) + SCAN_WARPS + 4;
  const size_t stage_bytes = (size_t)SCAN_CHUNK * slot * sizeof(float);
  int stages = (int)((44 * 1024) / stage_bytes);
  stages = stages > SCAN_MAX_STAGES ? SCAN_MAX_STAGES : stages;
  EL_REFUSE(stages >= 2, "ssm_scan: a state of %d rows does not leave room for two stages of inputs", N);
#define EL_SCAN(NK) do { if (N == 32 * NK) launch_pdl(pdl_bit_for_tokens(n_tokens), ssm_scan_kernel<NK, true>, dim3(grid), dim3(block), (size_t)(stages * stage_bytes), stream, xbc, C, inner, G, N, u, ldu, dta, Dp, state, y, seq_tok0, seq_slot, H, P, conv_state, conv_off, taps, vec, stages); \
    else launch_pdl(pdl_bit_for_tokens(n_tokens), ssm_scan_kernel<NK, false>, dim3(grid), dim3(block), (size_t)(stages * stage_bytes), stream, xbc, C, inner, G, N, u, ldu, dta, Dp, state, y, seq_tok0, seq_slot, H, P, conv_state, conv_off, taps, vec, stages); } while (0)
  if (N <= 32) EL_SCAN(1);
  else if (N <= 64) EL_SCAN(2);
  else if (N <= 128) EL_SCAN(4);
  else EL_SCAN(8);
#undef EL_SCAN
  EL_LAUNCH_CHECK("ssm_scan");
  return 0;
}

extern "C" int edgelm_wkv_scan(const float* r, const float* k, const float* v, const float* w, const float* bonus, float* state,
                               float* o, const int32_t* seq_tok0, const int32_t* seq_slot, int n_seqs, int H, int K, int n_tokens,
                               cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  EL_REFUSE(n_seqs > 0 && H > 0, "wkv_scan: bad sizes");
  EL_REFUSE(K >= 1 && K <= 256, "wkv_scan: a head size of %d is not taken (1 to 256)", K);
  // a warp a column, whatever the block: with few (sequence, head) pairs, blocks of two warps spread the columns over more SMs
  const int warps = (long long)n_seqs * H * ((K + SCAN_WARPS - 1) / SCAN_WARPS) >= 2 * 148 ? SCAN_WARPS : 2;
  const dim3 grid(n_seqs * H, (K + warps - 1) / warps), block(warps * 32);
#define EL_SCAN(NK, U) launch_pdl(pdl_bit_for_tokens(n_tokens), wkv_scan_kernel<NK, U>, dim3(grid), dim3(block), (size_t)(0), stream, r, k, v, w, bonus, state, o, seq_tok0, seq_slot, H, K)
  if (K <= 32) EL_SCAN(1, 8);
  else if (K <= 64) EL_SCAN(2, 8);
  else if (K <= 128) EL_SCAN(4, 4);
  else EL_SCAN(8, 1);
#undef EL_SCAN
  EL_LAUNCH_CHECK("wkv_scan");
  return 0;
}

extern "C" int edgelm_lowrank_decay(const float* a, const void* w2, int w_dtype, const float* w0, float* out, int n_tokens, int C,
                                    int L, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && C > 0 && L > 0 && L <= 8192, "lowrank_decay: bad sizes C=%d L=%d", C, L);
  const size_t smem = (size_t)L * sizeof(float);
  if (w_dtype == DT_F32) launch_pdl(pdl_bit_for_tokens(n_tokens), lowrank_decay_kernel<float>, dim3(n_tokens), dim3(row_threads(C)), (size_t)(smem), stream, a, (const float*)w2, w0, out, C, L);
  else if (w_dtype == DT_BF16) launch_pdl(pdl_bit_for_tokens(n_tokens), lowrank_decay_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(row_threads(C)), (size_t)(smem), stream, a, (const __nv_bfloat16*)w2, w0, out, C, L);
  else EL_REFUSE(false, "lowrank_decay: unknown dtype code %d", w_dtype);
  EL_LAUNCH_CHECK("lowrank_decay");
  return 0;
}

extern "C" int edgelm_gated_group_norm(const float* y, const float* gate, int ldg, const float* w, void* out, int out_dtype,
                                       int n_tokens, int inner, int groups, float eps, int gate_first, int gate_sigmoid, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && inner > 0 && groups > 0 && inner % groups == 0, "gated_group_norm: %d values do not split into %d equal groups", inner, groups);
  // (few rows of many values: a block of 1,024 threads walks a row in a quarter of the trips to memory)
  const int gs = inner / groups;
  const dim3 grid(n_tokens, groups), block(gs >= 1024 ? ((long long)n_tokens * groups <= 64 ? 1024 : 256) : (gs >= 128 ? 128 : 32));
  if (out_dtype == DT_F32) launch_pdl(pdl_bit_for_tokens(n_tokens), gated_group_norm_kernel<float>, dim3(grid), dim3(block), (size_t)(0), stream, y, gate, ldg, w, (float*)out, inner, groups, eps, gate_first, gate_sigmoid);
  else if (out_dtype == DT_BF16) launch_pdl(pdl_bit_for_tokens(n_tokens), gated_group_norm_kernel<__nv_bfloat16>, dim3(grid), dim3(block), (size_t)(0), stream, y, gate, ldg, w, (__nv_bfloat16*)out, inner, groups, eps, gate_first, gate_sigmoid);
  else EL_REFUSE(false, "gated_group_norm: unknown dtype code %d", out_dtype);
  EL_LAUNCH_CHECK("gated_group_norm");
  return 0;
}

// x += rmsnorm(a y1 + b y2) * w; y2 may be null; `xc` (may be null) receives x in `cast_dtype` as well.
extern "C" int edgelm_rmsnorm_add(float* x, const float* y1, float a, const float* y2, float b, const float* w, void* xc, int cast_dtype,
                                  int n_tokens, int dim, float eps, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && dim > 0, "rmsnorm_add: bad sizes");
  const dim3 grid(n_tokens), block(row_threads(dim));
  if (xc == nullptr || cast_dtype == DT_F32) launch_pdl(pdl_bit_for_tokens(n_tokens), rmsnorm_add_kernel<float>, dim3(grid), dim3(block), (size_t)(0), stream, x, y1, a, y2, b, w, (float*)xc, dim, eps);
  else if (cast_dtype == DT_BF16) launch_pdl(pdl_bit_for_tokens(n_tokens), rmsnorm_add_kernel<__nv_bfloat16>, dim3(grid), dim3(block), (size_t)(0), stream, x, y1, a, y2, b, w, (__nv_bfloat16*)xc, dim, eps);
  else EL_REFUSE(false, "rmsnorm_add: unknown dtype code %d", cast_dtype);
  EL_LAUNCH_CHECK("rmsnorm_add");
  return 0;
}
