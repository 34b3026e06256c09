// A feed-forward made of experts, of which every token uses the `top` with the largest router logits.
//
//   route     logits z = Wr h + br in float32 (a block a token); the `top` largest (first maximum on ties), and their
//             weights: the softmax over the chosen logits only.
//   route_scored   another router on the same logits: scores s = softmax(z) over all experts; the choice looks at s + a
//             correction per expert, optionally only inside the `keep` groups of neighbouring experts whose best corrected
//             score is largest; the weights are the chosen experts' s over their sum, times a constant.  The last experts may
//             be "identity experts" without weights (they give back their input): their pairs get no row, and `combine`
//             adds the token's own input for them.  Extra router rows after the experts give per-token gates (sigmoid).
//   plan      the (token, choice) pairs are grouped by expert: rows of a padded layout in which every expert's rows
//             start at a multiple of the row tile, so that a tile of rows belongs to one expert.
//             row_pair[row] = pair (token * top + choice) or -1; pair_row[pair] = its row; tile_expert[tile] = expert or -1.
//   products  mid[row] = silu(Wg_e h) * (Wu_e h) for the row's token; y[row] = Wd_e mid[row] (float32): on the CUDA
//             cores here (float32 models, sizes the tensor-core kernel does not take), or by the grouped tcgen05 product
//             over rows gathered by `gather_rows` (row tiles of 128).
//   combine   x[t] += sum_k weight[t][k] * y[pair_row[t * top + k]], in the order of k.
// Every row is computed by itself, so a token's result does not depend on what else is in the step.
#include "common.cuh"

namespace edgelm {

constexpr int MOE_MAX_EXPERTS = 1024;

// The router's logits of one token into shared memory: z[e] = wr[e] . h (+ br[e]).  A block a token: its four warps share the
// width, eight experts at a time (the token's row is read once for the eight, and a thread has eight independent sums and
// several steps of loads in flight); the warps' sums are added in a fixed order.  `part`: 32 floats.
template <typename TH>
__device__ __forceinline__ void moe_logits(const TH* __restrict__ row, const float* __restrict__ wr, const float* __restrict__ br,
                                           float* z, float* part, int D, int E) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int e0 = 0; e0 < E; e0 += 8) {
    const float* w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = wr + (size_t)min(e0 + j, E - 1) * D;     // (past the last expert: computed, not kept)
    float acc[8] = {};
#pragma unroll 4
    for (int i = threadIdx.x; i < D; i += 128) {
      const float x = to_f32(row[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(x, w[j][i], acc[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sj = warp_sum(acc[j]);
      if (lane == 0) part[warp * 8 + j] = sj;
    }
    __syncthreads();
    if (threadIdx.x < 8 && e0 + threadIdx.x < E)
      z[e0 + threadIdx.x] = ((part[threadIdx.x] + part[8 + threadIdx.x]) + (part[16 + threadIdx.x] + part[24 + threadIdx.x])) +
                            (br ? br[e0 + threadIdx.x] : 0.f);
    __syncthreads();
  }
}

template <typename TH>
__global__ void __launch_bounds__(128)
moe_route_kernel(const TH* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ br, int32_t* __restrict__ idx,
                 float* __restrict__ wts, int n_tokens, int D, int E, int top) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float mr_smem[];         // [E] logits, then [4][8] partial sums
  float* z = mr_smem;
  moe_logits(h + (size_t)blockIdx.x * D, wr, br, z, mr_smem + E, D, E);
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    float zmax = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
      int best = -1;
      float bz = -INFINITY;
      for (int e = 0; e < E; ++e)
        if (z[e] > bz) { bz = z[e]; best = e; }
      if (best < 0) best = 0;     // (every logit was NaN or -inf)
      if (k == 0) zmax = bz;
      const float p = expf(bz - zmax);
      idx[(size_t)t * top + k] = best;
      wts[(size_t)t * top + k] = p;
      sum += p;
      z[best] = -INFINITY;
    }
    const float inv = 1.0f / sum;
    for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] *= inv;
  }
}

// The scored router (see the head of this file).  E experts in all (the last ones may be identity experts: nothing here
// treats them differently), `n_extra` more router rows whose sigmoid goes to extra[t][.].  Ties: the first of equal scores.
template <typename TH>
__global__ void __launch_bounds__(128)
moe_route_scored_kernel(const TH* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ correction,
                        int32_t* __restrict__ idx, float* __restrict__ wts, float* __restrict__ extra, int D, int E, int n_extra, int top,
                        int groups, int keep, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float mr_smem[];         // [E + n_extra] logits, [E] choice scores, [groups] group scores, then [4][8] partial sums
  float* z = mr_smem;
  float* c = z + E + n_extra;
  float* gs = c + E;
  const int t = blockIdx.x;
  moe_logits(h + (size_t)t * D, wr, (const float*)nullptr, z, gs + groups, D, E + n_extra);
  if (threadIdx.x < n_extra) extra[(size_t)t * n_extra + threadIdx.x] = 1.0f / (1.0f + expf(-z[E + threadIdx.x]));
  if (threadIdx.x == 0) {
    float zmax = -INFINITY, sum = 0.f;
    for (int e = 0; e < E; ++e) zmax = fmaxf(zmax, z[e]);
    for (int e = 0; e < E; ++e) {
      z[e] = expf(z[e] - zmax);
      sum += z[e];
    }
    const float inv = 1.0f / sum;
    for (int e = 0; e < E; ++e) {
      z[e] *= inv;                                  // the score
      c[e] = z[e] + (correction ? correction[e] : 0.f);   // what the choice looks at
    }
    if (groups > 1) {
      const int size = E / groups;
      for (int g = 0; g < groups; ++g) {
        float b = -INFINITY;
        for (int e = g * size; e < (g + 1) * size; ++e) b = fmaxf(b, c[e]);
        gs[g] = b;
      }
      // a group is kept if fewer than `keep` groups come before it in the order (score descending, then index)
      for (int g = 0; g < groups; ++g) {
        int before = 0;
        for (int o = 0; o < groups; ++o) before += (gs[o] > gs[g] || (gs[o] == gs[g] && o < g)) ? 1 : 0;
        if (before >= keep)
          for (int e = g * size; e < (g + 1) * size; ++e) c[e] = -INFINITY;
      }
    }
    float picked = 0.f;
    for (int k = 0; k < top; ++k) {
      int best = -1;
      float bc = -INFINITY;
      for (int e = 0; e < E; ++e)
        if (c[e] > bc) { bc = c[e]; best = e; }
      if (best < 0)         // fewer allowed experts than `top`: the left-out ones follow in the order of their numbers
        for (int e = 0; e < E && best < 0; ++e)
          if (c[e] == -INFINITY) best = e;
      if (best < 0) {       // (nothing left at all: NaN scores)
        idx[(size_t)t * top + k] = -1;
        wts[(size_t)t * top + k] = 0.f;
        continue;
      }
      idx[(size_t)t * top + k] = best;
      wts[(size_t)t * top + k] = z[best];
      picked += z[best];
      c[best] = NAN;        // taken (compares false with everything; a left-out expert stays at minus infinity)
    }
    const float norm = scale / (picked + 1e-20f);
    for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] *= norm;
  }
}

// One block.  counts -> padded offsets -> rows.  The order of an expert's rows depends on the order in which the threads
// arrive; no result does, since every row is computed by itself.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int32_t* __restrict__ idx, int n_pairs, int E, int tile_rows, int max_tiles, int32_t* __restrict__ row_pair,
                int32_t* __restrict__ pair_row, int32_t* __restrict__ tile_expert) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int counts[MOE_MAX_EXPERTS], offs[MOE_MAX_EXPERTS];
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  for (int i = threadIdx.x; i < max_tiles * tile_rows; i += blockDim.x) row_pair[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = idx[i];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tile = 0;
    for (int e = 0; e < E; ++e) {
      offs[e] = tile * tile_rows;
      const int nt = (counts[e] + tile_rows - 1) / tile_rows;
      for (int j = 0; j < nt && tile < max_tiles; ++j) tile_expert[tile++] = e;
      counts[e] = 0;
    }
    for (; tile < max_tiles; ++tile) tile_expert[tile] = -1;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = idx[i];
    if (e >= 0 && e < E) {
      const int r = offs[e] + atomicAdd(&counts[e], 1);
      if (r < max_tiles * tile_rows) { row_pair[r] = i; pair_row[i] = r; }
    } else {
      pair_row[i] = -1;
    }
  }
}

// a[row][:] = h[row_pair[row] / top][:], zeros for a row of no pair: the grouped rows as a matrix of their own
template <typename T>
__global__ void moe_gather_rows_kernel(const T* __restrict__ h, T* __restrict__ a, const int32_t* __restrict__ row_pair, int top, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, p = row_pair[r];
  T* dst = a + (size_t)r * D;
  if (p < 0) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = from_f32<T>(0.f);
    return;
  }
  const T* src = h + (size_t)(p / top) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = src[i];
}

// The products on the CUDA cores (float32 sums): tiles of 32 rows x 64 columns, K in steps of 32 through shared memory.
//   GATED: a[row] = h[row_pair[row] / top]; out[row][n] = silu(a . wg_e[n]) * (a . wu_e[n])          (mid, type T)
//   else:  a[row] = mid[row];               y[row][n] = a . w_e[n]                                    (float32)
constexpr int MG_TM = 32, MG_TN = 64, MG_KC = 32;

template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ a, int lda, const T* __restrict__ w, const T* __restrict__ w2, void* __restrict__ out, int ldo,
                const int32_t* __restrict__ row_pair, const int32_t* __restrict__ tile_expert, int top, int K, int N, float glu_limit,
                float glu_alpha, float glu_shift) {
  pdl_launch_dependents();
  pdl_wait();
  const int e = tile_expert[blockIdx.x];
  if (e < 0) return;
  __shared__ float As[MG_TM][MG_KC + 1];
  __shared__ float Ws[MG_TN][MG_KC + 1];
  __shared__ float W2s[GATED ? MG_TN : 1][MG_KC + 1];
  __shared__ int pair_of[MG_TM];
  const int r0 = blockIdx.x * MG_TM, n0 = blockIdx.y * MG_TN;
  if (threadIdx.x < MG_TM) pair_of[threadIdx.x] = row_pair[r0 + threadIdx.x];
  __syncthreads();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const T* we = w + (size_t)e * N * K;
  const T* w2e = GATED ? w2 + (size_t)e * N * K : nullptr;
  float acc[2][4] = {}, acc2[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += MG_KC) {
    for (int i = threadIdx.x; i < MG_TM * MG_KC; i += 256) {
      const int r = i / MG_KC, k = i - r * MG_KC;
      const int p = pair_of[r];
      float v = 0.f;
      if (p >= 0 && k0 + k < K) v = to_f32(a[(size_t)(GATED ? p / top : r0 + r) * lda + k0 + k]);
      As[r][k] = v;
    }
    for (int i = threadIdx.x; i < MG_TN * MG_KC; i += 256) {
      const int r = i / MG_KC, k = i - r * MG_KC;
      const bool in = n0 + r < N && k0 + k < K;
      Ws[r][k] = in ? to_f32(we[(size_t)(n0 + r) * K + k0 + k]) : 0.f;
      if (GATED) W2s[r][k] = in ? to_f32(w2e[(size_t)(n0 + r) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < MG_KC; ++k) {
      const float a0 = As[ty * 2][k], a1 = As[ty * 2 + 1][k];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float wv = Ws[tx + 16 * j][k];
        acc[0][j] = fmaf(a0, wv, acc[0][j]);
        acc[1][j] = fmaf(a1, wv, acc[1][j]);
        if (GATED) {
          const float w2v = W2s[tx + 16 * j][k];
          acc2[0][j] = fmaf(a0, w2v, acc2[0][j]);
          acc2[1][j] = fmaf(a1, w2v, acc2[1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i, p = pair_of[r];
    if (p < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n >= N) continue;
      if (GATED) {
        // the gated unit: g sigmoid(alpha g) (v + shift), both branches clamped when there is a limit (none, 1, 0: SwiGLU)
        float z = acc[i][j], v = acc2[i][j];
        if (glu_limit > 0.f) {
          z = fminf(z, glu_limit);
          v = fminf(fmaxf(v, -glu_limit), glu_limit);
        }
        ((T*)out)[(size_t)(r0 + r) * ldo + n] = from_f32<T>(z / (1.0f + expf(-glu_alpha * z)) * (v + glu_shift));
      } else {
        ((float*)out)[(size_t)(r0 + r) * ldo + n] = acc[i][j];
      }
    }
  }
}

// x[t][:] += sum_k wts[t][k] * y[pair_row[t * top + k]][:]  (+ gate[t] * shared[t][:])
// A pair without a row whose expert number is at least `n_real` is an identity expert's: its output is the token's own input
// h[t] (in the type the experts read it in).
template <typename TH>
__global__ void moe_combine_kernel(float* __restrict__ x, const float* __restrict__ y, int ldy, const float* __restrict__ wts,
                                   const int32_t* __restrict__ pair_row, int top, int D, const int32_t* __restrict__ idx, int n_real,
                                   const TH* __restrict__ h, const float* __restrict__ shared, const float* __restrict__ gate) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int r = pair_row[(size_t)t * top + k];
      if (r >= 0) acc = fmaf(wts[(size_t)t * top + k], y[(size_t)r * ldy + i], acc);
      else if (idx && idx[(size_t)t * top + k] >= n_real) acc = fmaf(wts[(size_t)t * top + k], to_f32(h[(size_t)t * D + i]), acc);
    }
    if (shared) acc = fmaf(gate ? gate[t] : 1.0f, shared[(size_t)t * D + i], acc);
    x[(size_t)t * D + i] += acc;
  }
}

}  // namespace edgelm

using namespace edgelm;

extern "C" int edgelm_moe_tile_rows() { return MG_TM; }

extern "C" int edgelm_moe_route(const void* h, int dtype, const float* wr, const float* br, int32_t* idx, float* wts, int n_tokens, int D,
                                int E, int top, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && D > 0 && E >= 1 && E <= MOE_MAX_EXPERTS && top >= 1 && top <= E, "moe_route: %d experts, %d chosen", E, top);
  const dim3 grid(n_tokens), block(128);
  const size_t smem = (size_t)(E + 32) * sizeof(float);
  const int bit = pdl_bit_for_tokens(n_tokens);
  if (dtype == DT_F32) launch_pdl(bit, moe_route_kernel<float>, grid, block, smem, stream, (const float*)h, wr, br, idx, wts, n_tokens, D, E, top);
  else if (dtype == DT_BF16) launch_pdl(bit, moe_route_kernel<__nv_bfloat16>, grid, block, smem, stream, (const __nv_bfloat16*)h, wr, br, idx, wts, n_tokens, D, E, top);
  else EL_REFUSE(false, "moe_route: unknown dtype code %d", dtype);
  EL_LAUNCH_CHECK("moe_route");
  return 0;
}

extern "C" int edgelm_moe_route_scored(const void* h, int dtype, const float* wr, const float* correction, int32_t* idx, float* wts,
                                       float* extra, int n_tokens, int D, int E, int n_extra, int top, int groups, int keep, float scale,
                                       cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && D > 0 && E >= 1 && E <= MOE_MAX_EXPERTS && top >= 1 && top <= E, "moe_route_scored: %d experts, %d chosen", E, top);
  EL_REFUSE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups, "moe_route_scored: %d experts in %d groups, %d kept", E, groups, keep);
  EL_REFUSE(n_extra >= 0 && n_extra <= 32 && (n_extra == 0 || extra != nullptr), "moe_route_scored: %d extra rows (up to 32)", n_extra);
  const dim3 grid(n_tokens), block(128);
  const size_t smem = (size_t)(2 * E + n_extra + groups + 32) * sizeof(float);
  const int bit = pdl_bit_for_tokens(n_tokens);
  if (dtype == DT_F32) launch_pdl(bit, moe_route_scored_kernel<float>, grid, block, smem, stream, (const float*)h, wr, correction, idx, wts, extra, D, E, n_extra, top, groups, keep, scale);
  else if (dtype == DT_BF16) launch_pdl(bit, moe_route_scored_kernel<__nv_bfloat16>, grid, block, smem, stream, (const __nv_bfloat16*)h, wr, correction, idx, wts, extra, D, E, n_extra, top, groups, keep, scale);
  else EL_REFUSE(false, "moe_route_scored: unknown dtype code %d", dtype);
  EL_LAUNCH_CHECK("moe_route_scored");
  return 0;
}

extern "C" int edgelm_moe_plan(const int32_t* idx, int n_pairs, int E, int tile_rows, int max_tiles, int32_t* row_pair, int32_t* pair_row,
                               int32_t* tile_expert, cudaStream_t stream) {
  if (n_pairs == 0) return 0;
  EL_REFUSE(n_pairs > 0 && E >= 1 && E <= MOE_MAX_EXPERTS && tile_rows >= 1, "moe_plan: bad sizes");
  EL_REFUSE(max_tiles >= n_pairs / tile_rows + E || max_tiles >= n_pairs, "moe_plan: %d tiles of %d rows cannot hold %d pairs of %d experts", max_tiles, tile_rows, n_pairs, E);
  launch_pdl(pdl_bit_for_tokens(n_pairs), moe_plan_kernel, dim3(1), dim3(1024), (size_t)0, stream, idx, n_pairs, E, tile_rows, max_tiles, row_pair, pair_row, tile_expert);
  EL_LAUNCH_CHECK("moe_plan");
  return 0;
}

// gated != 0: the gate and up products with the activation; a = the tokens' rows [tokens][K]; out = mid [rows][N] in `dtype`.
// gated == 0: the down product; a = mid [rows][K]; out = y [rows][N] float32.
extern "C" int edgelm_moe_gemm(const void* a, int lda, const void* w, const void* w2, void* out, int ldo, const int32_t* row_pair,
                               const int32_t* tile_expert, int max_tiles, int top, int K, int N, int dtype, int gated, float glu_limit, float glu_alpha,
                               float glu_shift, cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  EL_REFUSE(max_tiles > 0 && K > 0 && N > 0 && top >= 1, "moe_gemm: bad sizes");
  const dim3 grid(max_tiles, (N + MG_TN - 1) / MG_TN), block(256);
  const int bit = pdl_bit_for_tokens(max_tiles);
#define EL_MG(T, GATED) launch_pdl(bit, moe_gemm_kernel<T, GATED>, grid, block, (size_t)0, stream, (const T*)a, lda, (const T*)w, (const T*)w2, out, ldo, row_pair, tile_expert, top, K, N, glu_limit, glu_alpha, glu_shift)
  if (dtype == DT_F32 && gated) EL_MG(float, true);
  else if (dtype == DT_F32) EL_MG(float, false);
  else if (dtype == DT_BF16 && gated) EL_MG(__nv_bfloat16, true);
  else if (dtype == DT_BF16) EL_MG(__nv_bfloat16, false);
  else EL_REFUSE(false, "moe_gemm: unknown dtype code %d", dtype);
#undef EL_MG
  EL_LAUNCH_CHECK("moe_gemm");
  return 0;
}

extern "C" int edgelm_moe_gather_rows(const void* h, void* a, const int32_t* row_pair, int n_rows, int top, int D, int dtype, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  EL_REFUSE(n_rows > 0 && top >= 1 && D > 0, "moe_gather_rows: bad sizes");
  const dim3 grid(n_rows), block(D >= 1024 ? 256 : 128);
  if (dtype == DT_F32) launch_pdl(pdl_bit_for_tokens(n_rows), moe_gather_rows_kernel<float>, grid, block, (size_t)0, stream, (const float*)h, (float*)a, row_pair, top, D);
  else if (dtype == DT_BF16) launch_pdl(pdl_bit_for_tokens(n_rows), moe_gather_rows_kernel<__nv_bfloat16>, grid, block, (size_t)0, stream, (const __nv_bfloat16*)h, (__nv_bfloat16*)a, row_pair, top, D);
  else EL_REFUSE(false, "moe_gather_rows: unknown dtype code %d", dtype);
  EL_LAUNCH_CHECK("moe_gather_rows");
  return 0;
}

// `idx`, `n_real`, `h` (type `h_dtype`): the experts' numbers, how many of them have weights, and the tokens' inputs, for identity
// experts (idx null: none).  `shared` [tokens][D] float32 with `gate` [tokens] (or null: 1): one more term for every token.
extern "C" int edgelm_moe_combine(float* x, const float* y, int ldy, const float* wts, const int32_t* pair_row, int n_tokens, int top, int D,
                                  const int32_t* idx, int n_real, const void* h, int h_dtype, const float* shared, const float* gate,
                                  cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && top >= 1 && D > 0 && ldy >= D && (idx == nullptr || h != nullptr), "moe_combine: bad sizes");
  const dim3 grid(n_tokens), block(D >= 1024 ? 256 : 128);
  const int bit = pdl_bit_for_tokens(n_tokens);
  if (h_dtype == DT_BF16) launch_pdl(bit, moe_combine_kernel<__nv_bfloat16>, grid, block, (size_t)0, stream, x, y, ldy, wts, pair_row, top, D, idx, n_real, (const __nv_bfloat16*)h, shared, gate);
  else launch_pdl(bit, moe_combine_kernel<float>, grid, block, (size_t)0, stream, x, y, ldy, wts, pair_row, top, D, idx, n_real, (const float*)h, shared, gate);
  EL_LAUNCH_CHECK("moe_combine");
  return 0;
}
