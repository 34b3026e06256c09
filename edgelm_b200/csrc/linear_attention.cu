// Linear attention with a constant decay per head ("lightning attention"): per head, with key size K and value size E,
//
//   S_t = decay_h S_(t-1) + k_t v_t^T          (S is K x E, float32, zero when a sequence starts)
//   o_t = S_t^T q_t                            (the read-out sees the token's own write)
//
// q, k, v are read from the float32 result of the stacked projection (row pitch ldu, column offsets q_off, k_off, v_off,
// head by head), after `silu_columns` has put them through their activation in place (or, with `act`, through silu as they are read).  Tokens of all sequences are packed along the first
// axis; `seq_tok0[s] .. seq_tok0[s + 1] - 1` are the packed rows of the step's sequence s, `seq_slot[s]` the row of its
// state [slot][H][E][K].  Everything is float32 in both precisions.
//
//   decay_scan     a warp owns one value channel j of one (sequence, head) and walks the sequence's tokens in order;
//                  lane l holds the key channels l, l + 32, ...  Any step: prompts, pieces of prompts, single tokens.
//   chunked form   for prompt steps: every sequence's rows of the step are cut into chunks of LC tokens (the step's tiles of
//                  that size), and the recurrence is rewritten chunk by chunk, with n the chunk's token count:
//                    1. `chunk_state`: every (chunk, head) sums its own tokens, A_c = sum_s decay^(n - 1 - s) k_s v_s^T;
//                    2. `chunk_fold`: per (sequence, head) the chunks in order: P_c = the state before chunk c (the slot's state
//                       for the first), S <- decay^n S + A_c; P_c replaces A_c, and the slot receives the last S;
//                    3. `chunk_out`: every (chunk, head): o_t = decay^(t + 1) P_c^T q_t + sum_(s <= t) decay^(t - s) (q_t . k_s) v_s.
//                  Powers of the decay come from a table that the host computed in double precision.  Every sum runs in a fixed order over
//                  the sequence's own rows, so a result does not depend on what else the step holds.  The activation is applied
//                  while the rows are staged (no pass of its own).
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

__device__ __forceinline__ float scan_silu(float z) { return z / (1.0f + expf(-z)); }

template <int NK, int U>
__global__ void __launch_bounds__(LA_WARPS * 32)
decay_scan_kernel(const float* __restrict__ u, int ldu, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                  float* __restrict__ state, float* __restrict__ o, const int32_t* __restrict__ seq_tok0,
                  const int32_t* __restrict__ seq_slot, int H, int K, int E, int act) {
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
        // (`act`: silu here instead of a pass of its own; every warp of a head repeats it for the keys and queries, which
        // costs less than a launch when a sequence brings one token)
        const float vj = act ? scan_silu(in.vj[x]) : in.vj[x];
#pragma unroll
        for (int k = 0; k < NK; ++k) {
          const float kv = act ? scan_silu(in.kk[x][k]) : in.kk[x][k], qv = act ? scan_silu(in.qq[x][k]) : in.qq[x][k];
          S[k] = fmaf(a, S[k], kv * vj);
          acc[x] = fmaf(S[k], qv, acc[x]);
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


// ------------------------------------------------------------------ the chunked form
constexpr int LC = 64;          // tokens of a chunk
constexpr int LC_THREADS = 256;

__device__ __forceinline__ float lc_act(float z, int act) { return act ? z / (1.0f + expf(-z)) : z; }

// decay^0 .. decay^LC of the block's head into shared memory, from the table [H][LC + 1] that the host made in double precision
__device__ __forceinline__ void lc_powers(float* pw, const float* __restrict__ table) {
  for (int n = threadIdx.x; n <= LC; n += blockDim.x) pw[n] = table[n];
}

// rows [ntok][n] of u from column `off` (row pitch ldu) into dst [LC][pitch], through the activation; rows past ntok are zero.
// A thread requests four pieces before it uses the first (a piece: 16 bytes where `vec` says the rows allow it), so that a
// block has a few thousand bytes on their way at once: one piece a thread at a time left the kernels waiting on memory.
__device__ __forceinline__ void lc_stage(float* dst, int pitch, const float* __restrict__ u, int ldu, int off, int tok0, int ntok, int n, int act, bool vec) {
  if (vec) {
    const int nv = n >> 2, total = LC * nv;
    for (int base = threadIdx.x; base < total; base += blockDim.x * 4) {
      float4 v[4];
      int at[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int idx = base + x * blockDim.x, r = idx / nv, c = (idx - r * nv) * 4;
        at[x] = idx < total ? r * pitch + c : -1;
        v[x] = idx < total && r < ntok ? *reinterpret_cast<const float4*>(u + (size_t)(tok0 + r) * ldu + off + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int x = 0; x < 4; ++x)
        if (at[x] >= 0) {
          dst[at[x]] = lc_act(v[x].x, act); dst[at[x] + 1] = lc_act(v[x].y, act);
          dst[at[x] + 2] = lc_act(v[x].z, act); dst[at[x] + 3] = lc_act(v[x].w, act);
        }
    }
    return;
  }
  const int total = LC * n;
  for (int base = threadIdx.x; base < total; base += blockDim.x * 4) {
    float v[4];
    int at[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int idx = base + x * blockDim.x, r = idx / n, c = idx - r * n;
      at[x] = idx < total ? r * pitch + c : -1;
      v[x] = idx < total && r < ntok ? u[(size_t)(tok0 + r) * ldu + off + c] : 0.f;
    }
#pragma unroll
    for (int x = 0; x < 4; ++x)
      if (at[x] >= 0) dst[at[x]] = lc_act(v[x], act);
  }
}

// whether rows of n floats from column `off` of u can be read 16 bytes at a time
__device__ __forceinline__ bool lc_vec_ok(const float* u, int ldu, int off, int n) {
  return ((n | off | ldu) & 3) == 0 && (reinterpret_cast<uintptr_t>(u) & 15) == 0;
}

// A small matrix product out of shared memory in registers: 256 threads as 16 x 16, thread (ty, tx) holds the sums of rows
// m0 + ty + 16 a (a < 4) and columns tx + 16 b (b < RN):  acc[a][b] += sum_(k < Kd) A(m, k) B(k, n)  with A(m, k) = a[m sam + k sak]
// and B(k, n) = b[k sbk + n sbn].  Rows and columns past M and N are computed on the last valid one and dropped by the caller.
// A warp reads two distinct A values (broadcast) and 16 B values a step: pitches are odd, so no bank is asked twice.
template <int RN>
__device__ __forceinline__ void lc_mm(float (&acc)[4][RN], const float* a, int sam, int sak, const float* b, int sbk, int sbn,
                                      int m0, int M, int N, int Kd) {
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  int am[4], bn[RN];
#pragma unroll
  for (int x = 0; x < 4; ++x) am[x] = min(m0 + ty + 16 * x, M - 1) * sam;
#pragma unroll
  for (int y = 0; y < RN; ++y) bn[y] = min(tx + 16 * y, N - 1) * sbn;
#pragma unroll 4
  for (int k = 0; k < Kd; ++k) {
    float av[4], bv[RN];
#pragma unroll
    for (int x = 0; x < 4; ++x) av[x] = a[am[x] + k * sak];
#pragma unroll
    for (int y = 0; y < RN; ++y) bv[y] = b[bn[y] + k * sbk];
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < RN; ++y) acc[x][y] = fmaf(av[x], bv[y], acc[x][y]);
  }
}

// 1. A[tile][h][j][i] = sum_s decay^(ntok - 1 - s) k_s[i] v_s[j]
template <int RN>      // RN = ceil(K / 16)
__global__ void __launch_bounds__(LC_THREADS)
decay_chunk_state_kernel(const float* __restrict__ u, int ldu, int k_off, int v_off, const float* __restrict__ powers, float* __restrict__ A,
                         const int32_t* __restrict__ tile_tok0, const int32_t* __restrict__ tile_ntok, int H, int K, int E, int act) {
  extern __shared__ float lc_smem[];
  float* ks = lc_smem;                    // [LC][K + 1], scaled by the power of the decay that the row still meets
  float* vs = ks + LC * (K + 1);          // [LC][E + 1]
  float* pw = vs + LC * (E + 1);          // [LC + 1]
  const int tile = blockIdx.x, h = blockIdx.y;
  const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
  lc_powers(pw, powers + (size_t)h * (LC + 1));
  lc_stage(ks, K + 1, u, ldu, k_off + h * K, tok0, ntok, K, act, lc_vec_ok(u, ldu, k_off + h * K, K));
  lc_stage(vs, E + 1, u, ldu, v_off + h * E, tok0, ntok, E, act, lc_vec_ok(u, ldu, v_off + h * E, E));
  __syncthreads();
  for (int i = threadIdx.x; i < ntok * K; i += blockDim.x) {
    const int r = i / K, c = i - r * K;
    ks[r * (K + 1) + c] *= pw[ntok - 1 - r];
  }
  __syncthreads();
  float* out = A + ((size_t)tile * H + h) * E * K;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  for (int j0 = 0; j0 < E; j0 += 64) {          // rows: value channels j; columns: key channels i; summed over the chunk's tokens
    float acc[4][RN] = {};
    lc_mm<RN>(acc, vs, 1, E + 1, ks, K + 1, 1, j0, E, K, ntok);
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < RN; ++y) {
        const int j = j0 + ty + 16 * x, i = tx + 16 * y;
        if (j < E && i < K) out[(size_t)j * K + i] = acc[x][y];
      }
  }
}

// 2. per (sequence, head), element by element: the chunks in order; P_c overwrites A_c, the slot's state moves on.  A thread
// an element; it requests eight chunks' values before the chain of multiply-adds through them (the values do not depend on it).
__global__ void decay_chunk_fold_kernel(float* __restrict__ A, float* __restrict__ state, const float* __restrict__ powers,
                                        const int32_t* __restrict__ seq_tok0, const int32_t* __restrict__ seq_slot, int H, int KE) {
  const int s = blockIdx.x / H, h = blockIdx.x - s * H;
  const int o = blockIdx.y * blockDim.x + threadIdx.x;
  if (o >= KE) return;
  int first = 0;                                                    // the sequence's first tile: every earlier sequence has ceil(n / LC)
  for (int p = 0; p < s; ++p) first += (seq_tok0[p + 1] - seq_tok0[p] + LC - 1) / LC;
  const int n = seq_tok0[s + 1] - seq_tok0[s], chunks = (n + LC - 1) / LC;
  if (chunks == 0) return;
  const float full = powers[(size_t)h * (LC + 1) + LC], last = powers[(size_t)h * (LC + 1) + n - (chunks - 1) * LC];
  float* sp = state + ((size_t)seq_slot[s] * H + h) * KE + o;
  float* a = A + ((size_t)first * H + h) * KE + o;
  const size_t step = (size_t)H * KE;
  float S = *sp;
  for (int c0 = 0; c0 < chunks; c0 += 8) {
    float add[8];
#pragma unroll
    for (int x = 0; x < 8; ++x) add[x] = c0 + x < chunks ? a[(size_t)(c0 + x) * step] : 0.f;
#pragma unroll
    for (int x = 0; x < 8; ++x)
      if (c0 + x < chunks) {
        a[(size_t)(c0 + x) * step] = S;
        S = fmaf(c0 + x + 1 < chunks ? full : last, S, add[x]);
      }
  }
  *sp = S;
}

// 3. o_t = decay^(t + 1) P^T q_t + sum_(s <= t) decay^(t - s) (q_t . k_s) v_s for the chunk's tokens
template <int RN>      // RN = ceil(E / 16)
__global__ void __launch_bounds__(LC_THREADS)
decay_chunk_out_kernel(const float* __restrict__ u, int ldu, int q_off, int k_off, int v_off, const float* __restrict__ powers,
                       const float* __restrict__ P, float* __restrict__ o, const int32_t* __restrict__ tile_tok0,
                       const int32_t* __restrict__ tile_ntok, int H, int K, int E, int act) {
  extern __shared__ float lc_smem[];
  float* qs = lc_smem;                    // [LC][K + 1]
  float* ks = qs + LC * (K + 1);          // [LC][K + 1]
  float* vs = ks + LC * (K + 1);          // [LC][E + 1]
  float* ps = vs + LC * (E + 1);          // [K][E + 1]   (P[i][j]: the state before the chunk)
  float* ws = ps + K * (E + 1);           // [LC][LC + 1] (the weights of the chunk's own tokens)
  float* pw = ws + LC * (LC + 1);         // [LC + 1]
  const int tile = blockIdx.x, h = blockIdx.y;
  const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  lc_powers(pw, powers + (size_t)h * (LC + 1));
  const float* pin = P + ((size_t)tile * H + h) * E * K;       // stored [j][i]
  for (int base = threadIdx.x; base < E * K; base += blockDim.x * 4) {      // (four requests a thread before the first is used)
    float v[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) v[x] = base + x * blockDim.x < E * K ? pin[base + x * blockDim.x] : 0.f;
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int idx = base + x * blockDim.x, j = idx / K, i = idx - j * K;
      if (idx < E * K) ps[i * (E + 1) + j] = v[x];
    }
  }
  lc_stage(qs, K + 1, u, ldu, q_off + h * K, tok0, ntok, K, act, lc_vec_ok(u, ldu, q_off + h * K, K));
  lc_stage(ks, K + 1, u, ldu, k_off + h * K, tok0, ntok, K, act, lc_vec_ok(u, ldu, k_off + h * K, K));
  lc_stage(vs, E + 1, u, ldu, v_off + h * E, tok0, ntok, E, act, lc_vec_ok(u, ldu, v_off + h * E, E));
  __syncthreads();
  {   // the chunk's own weights: w[t][r] = decay^(t - r) (q_t . k_r) for r <= t, else 0
    float acc[4][4] = {};
    lc_mm<4>(acc, qs, K + 1, 1, ks, 1, K + 1, 0, LC, LC, K);
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const int t = ty + 16 * x, r = tx + 16 * y;
        ws[t * (LC + 1) + r] = r <= t ? acc[x][y] * pw[t - r] : 0.f;
      }
  }
  __syncthreads();
  float acc[4][RN] = {};
  lc_mm<RN>(acc, qs, K + 1, 1, ps, E + 1, 1, 0, LC, E, K);           // what the earlier chunks left: q_t . P[:, j]
#pragma unroll
  for (int x = 0; x < 4; ++x)
#pragma unroll
    for (int y = 0; y < RN; ++y) acc[x][y] *= pw[ty + 16 * x + 1];
  lc_mm<RN>(acc, ws, LC + 1, 1, vs, E + 1, 1, 0, LC, E, ntok);       // the chunk's own tokens
#pragma unroll
  for (int x = 0; x < 4; ++x)
#pragma unroll
    for (int y = 0; y < RN; ++y) {
      const int t = ty + 16 * x, j = tx + 16 * y;
      if (t < ntok && j < E) o[(size_t)(tok0 + t) * H * E + (size_t)h * E + j] = acc[x][y];
    }
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
                                 int act, cudaStream_t stream) {
  if (n_seqs == 0 || n_tokens == 0) return 0;
  EL_REFUSE(n_seqs > 0 && H > 0 && E > 0 && ldu > 0 && q_off >= 0 && k_off >= 0 && v_off >= 0, "decay_scan: bad sizes");
  EL_REFUSE(K >= 1 && K <= 256, "decay_scan: a key size of %d is not taken (1 to 256)", K);
  // a warp a value channel, whatever the block: with few (sequence, head) pairs, blocks of two warps spread the channels over more SMs
  const int warps = (long long)n_seqs * H * ((E + LA_WARPS - 1) / LA_WARPS) >= 2 * 148 ? LA_WARPS : 2;
  const dim3 grid(n_seqs * H, (E + warps - 1) / warps), block(warps * 32);
#define EL_SCAN(NK, U) launch_pdl(pdl_bit_for_tokens(n_tokens), decay_scan_kernel<NK, U>, dim3(grid), dim3(block), (size_t)(0), stream, u, ldu, q_off, k_off, v_off, decay, state, o, seq_tok0, seq_slot, H, K, E, act)
  if (n_tokens == n_seqs) {      // one token a sequence: no tokens to look ahead for
    if (K <= 32) EL_SCAN(1, 1);
    else if (K <= 64) EL_SCAN(2, 1);
    else if (K <= 128) EL_SCAN(4, 1);
    else EL_SCAN(8, 1);
  } else if (K <= 32) EL_SCAN(1, 8);
  else if (K <= 64) EL_SCAN(2, 8);
  else if (K <= 128) EL_SCAN(4, 4);
  else EL_SCAN(8, 1);
#undef EL_SCAN
  EL_LAUNCH_CHECK("decay_scan");
  return 0;
}

extern "C" int edgelm_decay_chunk_tokens() { return LC; }

// Floats of scratch that the chunked form takes for `n_tiles` chunks.
extern "C" long long edgelm_decay_chunked_scratch(int n_tiles, int H, int K, int E) { return (long long)n_tiles * H * K * E; }

// 1 if the chunked form takes these head sizes (its tiles must fit in shared memory).
extern "C" int edgelm_decay_chunked_takes(int K, int E) {
  const size_t smem = ((size_t)2 * LC * (K + 1) + (size_t)LC * (E + 1) + (size_t)K * (E + 1) + (size_t)LC * (LC + 1) + LC + 1) * sizeof(float);
  return K >= 1 && E >= 1 && K <= 128 && E <= 128 && smem <= 200 * 1024 ? 1 : 0;
}

// The step's tokens come as tiles of at most LC consecutive tokens of one sequence, in the order of the sequences, every
// sequence cut from its first row of the step (so sequence s has ceil(n_s / LC) tiles).  `act` != 0: q, k and v pass silu as they
// are read.  scratch: `edgelm_decay_chunked_scratch` floats.
// `powers` [H][LC + 1]: decay_h^0 .. decay_h^LC, each rounded once from double precision (the host makes the table with the decays).
extern "C" int edgelm_decay_chunked(const float* u, int ldu, int q_off, int k_off, int v_off, const float* powers, float* state, float* o,
                                    const int32_t* seq_tok0, const int32_t* seq_slot, int n_seqs, const int32_t* tile_tok0,
                                    const int32_t* tile_ntok, int n_tiles, int H, int K, int E, int act, float* scratch, cudaStream_t stream) {
  if (n_seqs == 0 || n_tiles == 0) return 0;
  EL_REFUSE(n_seqs > 0 && n_tiles > 0 && H > 0 && H <= 65535 && ldu > 0 && scratch != nullptr, "decay_chunked: bad sizes");
  EL_REFUSE(edgelm_decay_chunked_takes(K, E), "decay_chunked: heads of %d x %d do not fit (use the scan)", K, E);
  const size_t smem1 = ((size_t)LC * (K + 1) + (size_t)LC * (E + 1) + LC + 1) * sizeof(float);
  const size_t smem3 = ((size_t)2 * LC * (K + 1) + (size_t)LC * (E + 1) + (size_t)K * (E + 1) + (size_t)LC * (LC + 1) + LC + 1) * sizeof(float);
  auto k1 = K <= 64 ? decay_chunk_state_kernel<4> : decay_chunk_state_kernel<8>;
  auto k3 = E <= 64 ? decay_chunk_out_kernel<4> : decay_chunk_out_kernel<8>;
  if (smem1 > 48 * 1024) cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
  if (smem3 > 48 * 1024) cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
  k1<<<dim3(n_tiles, H), LC_THREADS, smem1, stream>>>(u, ldu, k_off, v_off, powers, scratch, tile_tok0, tile_ntok, H, K, E, act);
  EL_LAUNCH_CHECK("decay_chunk_state");
  const int KE = K * E;
  decay_chunk_fold_kernel<<<dim3(n_seqs * H, (KE + 127) / 128), 128, 0, stream>>>(scratch, state, powers, seq_tok0, seq_slot, H, KE);
  EL_LAUNCH_CHECK("decay_chunk_fold");
  k3<<<dim3(n_tiles, H), LC_THREADS, smem3, stream>>>(u, ldu, q_off, k_off, v_off, powers, scratch, o, tile_tok0, tile_ntok, H, K, E, act);
  EL_LAUNCH_CHECK("decay_chunk_out");
  return 0;
}
