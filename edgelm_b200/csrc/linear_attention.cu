// Linear attention with a constant decay per head ("lightning attention"): per head, with key size K and value size E,
//
//   S_t = decay_h S_(t-1) + k_t v_t^T          (S is K x E, float32, zero when a sequence starts)
//   o_t = S_t^T q_t                            (the read-out sees the token's own write)
//
// q, k, v are read from the float32 result of the stacked projection (row pitch ldu, column offsets q_off, k_off, v_off,
// head by head), after `silu_columns` has put them through their activation in place.  Tokens of all sequences are packed along the first
// axis; `seq_tok0[s] .. seq_tok0[s + 1] - 1` are the packed rows of the step's sequence s, `seq_slot[s]` the row of its
// state [slot][H][E][K].  Everything is float32 in both precisions.
//
//   decay_scan     a warp owns one value channel j of one (sequence, head) and walks the sequence's tokens in order;
//                  lane l holds the key channels l, l + 32, ...  Any step: prompts, pieces of prompts, single tokens.
#include "common.cuh"

namespace edgelm {

// u[t][off + c] <- silu(u[t][off + c]) for c < n: the activation of projections that feed the recurrence, once per element
// (the scan's warps would each compute it again for their value channel).
__global__ void silu_columns_kernel(float* __restrict__ u, int ldu, int off, int n) {
  pdl_launch_dependents();
  pdl_wait();
  float* row = u + (size_t)blockIdx.x * ldu + off;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x) {
    const float z = row[c];
    row[c] = z / (1.0f + expf(-z));
  }
}

template <int U>
__device__ __forceinline__ float la_warp_sums(float (&acc)[U], int lane) {
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

constexpr int LA_WARPS = 8;

template <int NK, int U>
__global__ void __launch_bounds__(LA_WARPS * 32)
decay_scan_kernel(const float* __restrict__ u, int ldu, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                  float* __restrict__ state, float* __restrict__ o, const int32_t* __restrict__ seq_tok0,
                  const int32_t* __restrict__ seq_slot, int H, int K, int E) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: nothing is read or written before the kernel ahead is done)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = blockIdx.x / H, h = blockIdx.x - s * H;
  const int j = blockIdx.y * (blockDim.x >> 5) + warp;
  if (j >= E) return;
  const int t0 = seq_tok0[s], t1 = seq_tok0[s + 1];
  float* sp = state + (((size_t)seq_slot[s] * H + h) * E + j) * K;
  const float a = decay[h];
  float S[NK];
#pragma unroll
  for (int k = 0; k < NK; ++k) S[k] = lane + 32 * k < K ? sp[lane + 32 * k] : 0.f;
  const float* qb = u + q_off + (size_t)h * K;
  const float* kb = u + k_off + (size_t)h * K;
  const float* vb = u + v_off + (size_t)h * E + j;
  struct Inputs { float vj[U], qq[U][NK], kk[U][NK]; };
  auto load = [&](int tb, Inputs& in) {
#pragma unroll
    for (int x = 0; x < U; ++x) {
      const size_t row = (size_t)min(tb + x, t1 - 1) * ldu;
      in.vj[x] = vb[row];
#pragma unroll
      for (int k = 0; k < NK; ++k) {
        const int i = lane + 32 * k;
        in.qq[x][k] = i < K ? qb[row + i] : 0.f;
        in.kk[x][k] = i < K ? kb[row + i] : 0.f;
      }
    }
  };
  auto compute = [&](int tb, const Inputs& in) {
    float acc[U];
#pragma unroll
    for (int x = 0; x < U; ++x) {
      acc[x] = 0.f;
      if (tb + x < t1) {
        const float vj = in.vj[x];
#pragma unroll
        for (int k = 0; k < NK; ++k) {
          S[k] = fmaf(a, S[k], in.kk[x][k] * vj);
          acc[x] = fmaf(S[k], in.qq[x][k], acc[x]);
        }
      }
    }
    const float sum = la_warp_sums<U>(acc, lane);
    const int x = lane / (32 / U);
    if ((lane & (32 / U - 1)) == 0 && tb + x < t1) o[(size_t)(tb + x) * H * E + (size_t)h * E + j] = sum;
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

}  // namespace edgelm

using namespace edgelm;

extern "C" int edgelm_silu_columns(float* u, int ldu, int off, int n, int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0 || n == 0) return 0;
  EL_REFUSE(n_tokens > 0 && n > 0 && off >= 0 && ldu >= off + n, "silu_columns: bad sizes");
  const dim3 grid(n_tokens, n_tokens >= 256 ? 1 : (n + 511) / 512), block(n >= 1024 ? 256 : 128);
  launch_pdl(pdl_bit_for_tokens(n_tokens), silu_columns_kernel, grid, block, (size_t)0, stream, u, ldu, off, n);
  EL_LAUNCH_CHECK("silu_columns");
  return 0;
}

extern "C" int edgelm_decay_scan(const float* u, int ldu, int q_off, int k_off, int v_off, const float* decay, float* state, float* o,
                                 const int32_t* seq_tok0, const int32_t* seq_slot, int n_seqs, int H, int K, int E, int n_tokens,
                                 cudaStream_t stream) {
  if (n_seqs == 0 || n_tokens == 0) return 0;
  EL_REFUSE(n_seqs > 0 && H > 0 && E > 0 && ldu > 0 && q_off >= 0 && k_off >= 0 && v_off >= 0, "decay_scan: bad sizes");
  EL_REFUSE(K >= 1 && K <= 256, "decay_scan: a key size of %d is not taken (1 to 256)", K);
  // a warp a value channel, whatever the block: with few (sequence, head) pairs, blocks of two warps spread the channels over more SMs
  const int warps = (long long)n_seqs * H * ((E + LA_WARPS - 1) / LA_WARPS) >= 2 * 148 ? LA_WARPS : 2;
  const dim3 grid(n_seqs * H, (E + warps - 1) / warps), block(warps * 32);
#define EL_SCAN(NK, U) launch_pdl(pdl_bit_for_tokens(n_tokens), decay_scan_kernel<NK, U>, dim3(grid), dim3(block), (size_t)(0), stream, u, ldu, q_off, k_off, v_off, decay, state, o, seq_tok0, seq_slot, H, K, E)
  if (K <= 32) EL_SCAN(1, 8);
  else if (K <= 64) EL_SCAN(2, 8);
  else if (K <= 128) EL_SCAN(4, 4);
  else EL_SCAN(8, 1);
#undef EL_SCAN
  EL_LAUNCH_CHECK("decay_scan");
  return 0;
}
