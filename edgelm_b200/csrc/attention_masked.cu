// Attention over the paged cache with a key range per query and an optional sink, for head sizes that the other
// attention kernels do not take, and the kernels that prepare its queries and keys.
//
// A query at position i sees the keys lo(i) .. i, where lo depends on the mask:
//   MASK_CAUSAL  lo = 0
//   MASK_WINDOW  lo = max(0, i - size + 1)                  (the last `size` keys)
//   MASK_CHUNK   lo = (i / size) * size                     (the keys of its own chunk of `size` positions)
// `sink` (optional, one float per query head): one more term exp(sink_h) in the softmax's denominator that has no key
// and no value and is not scaled.  Scores, maxima, exponentials, sums and weighted values are float32; queries come
// as float32, keys and values in the cache's type.
//
// Cache layout: keys [page][kv_head][PAGE][dk]; values either [page][kv_head][PAGE][dv] (a tensor of their own) or
// the first dv dimensions of each key row (`vcache` null: a latent that is key and value at once).
//
// Kernels: `rotate_append` (bias, rotation of a part of every query and key head with neighbouring or half-split
// pairs, cache append); `latent_prepare` (rotation of the queries' rotated part; RMS norm of the latent, rotation of
// the shared key part, cache append); `head_matmul` (one small matrix product per head: queries into the latent's
// space, weighted latents out of it); `masked_attn` (a block per token and head: steps of one token a sequence);
// `masked_attn_tiled` (prompt steps: keys staged once for 32 rows, from the cache's pages or from the step's own rows);
// `latent_expand_keys`; `add_row_bias`.
#include "common.cuh"

namespace edgelm {

enum : int { MASK_CAUSAL = 0, MASK_WINDOW = 1, MASK_CHUNK = 2 };

__device__ __forceinline__ int first_key(int pos, int mask, int size) {
  if (mask == MASK_WINDOW) return max(0, pos - size + 1);
  if (mask == MASK_CHUNK) return (pos / size) * size;
  return 0;
}

// sine and cosine of position * f: the product is formed in float64 and brought into [-pi, pi] before it is rounded
// (a float32 product alone is off by 3e-5 rad at position 1,000)
__device__ __forceinline__ void angle_sincos(double pos, double f, float* sn, float* cs) {
  double a = pos * f;
  a -= 6.283185307179586477 * rint(a * 0.15915494309189533577);
  sincosf((float)a, sn, cs);
}

// element i (< rot) of a rotated run x[0 .. rot): pairs (2j, 2j + 1) if `interleaved`, else (j, j + rot / 2)
__device__ __forceinline__ float rotated(const float* x, int i, int rot, int interleaved, double pos, const double* __restrict__ freq) {
  const int half = rot >> 1;
  int j, partner;
  bool first;
  if (interleaved) { j = i >> 1; first = (i & 1) == 0; partner = i ^ 1; }
  else { first = i < half; j = first ? i : i - half; partner = first ? i + half : i - half; }
  float sn, cs;
  angle_sincos(pos, freq[j], &sn, &cs);
  return first ? x[i] * cs - x[partner] * sn : x[i] * cs + x[partner] * sn;
}

constexpr int MA_WARPS = 4;

// qkv [tokens][H dk + G dk + G dv] float32 (+ bias): the first `rot` dimensions of every query and key head rotated;
// queries to q_out [tokens][H][dk] float32, keys and values into their cache rows.  A head may be `maps` runs of dk / maps
// dimensions side by side (the maps of a differential attention): then each run is rotated by itself.  With `q_norm` /
// `k_norm` (dk / maps weights each, shared by all heads and runs) every run is first divided by its root mean square
// (eps inside the root) and multiplied by the weight.
// With `conv_w` ([channels][taps], channels = the q | k | v columns) every channel first passes a causal filter over time,
// out_t[c] = sum_j w[c][j] in_(t - taps + 1 + j)[c] with in = qkv + bias; inputs from before the step come from `conv_state`
// [slot][taps - 1][channels] (oldest first; zeros before a sequence's start), so the projection's result goes through the
// filter, the norm, the rotation and into the cache without a trip to memory between.  `move_tail` (steps of one token a
// sequence only: the thread of a channel is then the only one that touches the sequence's tail of that channel): the tail
// moves on by the token's input here; other steps leave that to `conv_tail_update` afterwards.
struct ConvAhead {
  const float* w = nullptr;
  float* state = nullptr;
  const int32_t* seq_tok0 = nullptr;
  const int32_t* seq_slot = nullptr;
  int taps = 0, move_tail = 0;
};

template <typename T>
__global__ void __launch_bounds__(MA_WARPS * 32)
rotate_append_kernel(const float* __restrict__ qkv, const float* __restrict__ bias, float* __restrict__ q_out,
                     const int32_t* __restrict__ tok_pos, const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ page_table,
                     int table_stride, int n_pages, T* __restrict__ kcache, T* __restrict__ vcache, int H, int G, int dk, int dv,
                     int rot, int interleaved, const double* __restrict__ freq, int* __restrict__ err, int maps,
                     const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps, int ldq, ConvAhead conv) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float ra_stage[];   // MA_WARPS rows of dk floats
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = tok_pos[t];
  if (pos < 0) {
    if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, ERR_POSITION_RANGE);
    return;
  }
  const int page = page_table[(size_t)tok_seq[t] * table_stride + pos / PAGE];
  if (page < 0 || page >= n_pages) {
    if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, ERR_PAGE_RANGE);
    return;
  }
  const int in_page = pos % PAGE;
  const float* row = qkv + (size_t)t * ldq;       // (ldq: the rows' pitch; a row may hold more than q | k | v)
  float* sh = ra_stage + warp * dk;
  // channel c after the filter over time (and the tail moved on, if this thread is to do it)
  const int C = (H + G) * dk + G * dv;
  const int cs = conv.w ? tok_seq[t] : 0, ct0 = conv.w ? conv.seq_tok0[cs] : 0, ck = t - ct0;
  float* tail = conv.w ? conv.state + (size_t)conv.seq_slot[cs] * (conv.taps - 1) * C : nullptr;
  auto filtered = [&](int c) -> float {
    const float ib = bias ? bias[c] : 0.f;
    float acc = 0.f;
    for (int j = 0; j < conv.taps; ++j) {
      const int r = ck - (conv.taps - 1) + j;
      const float v = r >= 0 ? qkv[(size_t)(ct0 + r) * ldq + c] + ib : tail[(size_t)(conv.taps - 1 + r) * C + c];
      acc = fmaf(conv.w[(size_t)c * conv.taps + j], v, acc);
    }
    if (conv.move_tail && conv.taps > 1) {      // (every row of the tail was read above; row j takes row j + 1, the last one the token's input)
      for (int j = 0; j + 2 < conv.taps; ++j) tail[(size_t)j * C + c] = tail[(size_t)(j + 1) * C + c];
      tail[(size_t)(conv.taps - 2) * C + c] = row[c] + ib;
    }
    return acc;
  };
  for (int head = blockIdx.y * MA_WARPS + warp; head < H + G; head += gridDim.y * MA_WARPS) {
    const float* src = row + (size_t)head * dk;
    const float* b = bias ? bias + (size_t)head * dk : nullptr;
    if (conv.w) for (int i = lane; i < dk; i += 32) sh[i] = filtered(head * dk + i);
    else for (int i = lane; i < dk; i += 32) sh[i] = src[i] + (b ? b[i] : 0.f);
    __syncwarp();
    const int ds = dk / maps;
    const float* nw = head < H ? q_norm : k_norm;
    if (nw) {
      for (int mp = 0; mp < maps; ++mp) {
        float* run = sh + mp * ds;
        float ss = 0.f;
        for (int i = lane; i < ds; i += 32) ss = fmaf(run[i], run[i], ss);
        const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)ds + eps);
        for (int i = lane; i < ds; i += 32) run[i] = run[i] * inv * nw[i];
      }
      __syncwarp();
    }
    for (int i = lane; i < dk; i += 32) {
      const int mp = i / ds, j = i - mp * ds;
      const float x = j < rot ? rotated(sh + mp * ds, j, rot, interleaved, (double)pos, freq) : sh[i];
      if (head < H) q_out[((size_t)t * H + head) * dk + i] = x;
      else kcache[(((size_t)page * G + (head - H)) * PAGE + in_page) * dk + i] = from_f32<T>(x);
    }
    __syncwarp();
  }
  const float* vrow = row + (size_t)(H + G) * dk;
  const float* vb = bias ? bias + (size_t)(H + G) * dk : nullptr;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < G * dv; i += gridDim.y * blockDim.x) {
    const int g = i / dv, j = i - g * dv;
    vcache[(((size_t)page * G + g) * PAGE + in_page) * dv + j] = from_f32<T>(conv.w ? filtered((H + G) * dk + i) : vrow[i] + (vb ? vb[i] : 0.f));
  }
}

// u [tokens][ldu] float32: H query heads of [d | rd] from column 0 and, with `has_kv`, the latent's row [r | rd] from
// column kv_off.  The rotated part of every query head (half-split pairs) goes to q_out[t][h * q_pitch + q_off + i], and with
// `copy_q` the unrotated part to q_out[t][h * q_pitch + i]; the latent, divided by its root mean square and times `norm_w`,
// and the rotated shared key part become the token's cache row [r + rd] (one key head) and, if `row_out` is given, row t
// of it as well (what the cache holds, for a step that expands its own keys).
template <typename T>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ u, int ldu, int kv_off, int has_kv, float* __restrict__ q_out, int q_pitch, int q_off,
                      int copy_q, const float* __restrict__ norm_w, float eps, const int32_t* __restrict__ tok_pos,
                      const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ page_table, int table_stride, int n_pages,
                      T* __restrict__ kcache, T* __restrict__ row_out, int H, int d, int rd, int r, const double* __restrict__ freq,
                      int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  if (pos < 0) {
    if (threadIdx.x == 0) atomicOr(err, ERR_POSITION_RANGE);
    return;
  }
  const float* row = u + (size_t)t * ldu;
  float* qo = q_out + (size_t)t * H * q_pitch;
  for (int i = threadIdx.x; i < H * rd; i += blockDim.x) {
    const int h = i / rd, j = i - h * rd;
    qo[(size_t)h * q_pitch + q_off + j] = rotated(row + (size_t)h * (d + rd) + d, j, rd, 0, (double)pos, freq);
  }
  if (copy_q)
    for (int i = threadIdx.x; i < H * d; i += blockDim.x) {
      const int h = i / d, j = i - h * d;
      qo[(size_t)h * q_pitch + j] = row[(size_t)h * (d + rd) + j];
    }
  if (!has_kv) return;
  const int page = page_table[(size_t)tok_seq[t] * table_stride + pos / PAGE];
  if (page < 0 || page >= n_pages) {
    if (threadIdx.x == 0) atomicOr(err, ERR_PAGE_RANGE);
    return;
  }
  const float* c = row + kv_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < r; i += blockDim.x) ss = fmaf(c[i], c[i], ss);
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)r + eps);
  T* dst = kcache + ((size_t)page * PAGE + pos % PAGE) * (r + rd);
  T* dst2 = row_out ? row_out + (size_t)t * (r + rd) : nullptr;
  for (int i = threadIdx.x; i < r + rd; i += blockDim.x) {
    const T v = from_f32<T>(i < r ? c[i] * inv * norm_w[i] : rotated(c + r, i - r, rd, 0, (double)pos, freq));
    dst[i] = v;
    if (dst2) dst2[i] = v;
  }
}

// kx[t][h][:] = [kn[t][h][0 .. d) | row[t][r .. r + rd)]: a step's keys per head, the shared rotated part repeated
template <typename T>
__global__ void latent_expand_keys_kernel(const T* __restrict__ kn, const T* __restrict__ rows, T* __restrict__ kx, int H, int d, int rd, int r) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* shared_part = rows + (size_t)t * (r + rd) + r;
  for (int i = threadIdx.x; i < H * (d + rd); i += blockDim.x) {
    const int h = i / (d + rd), j = i - h * (d + rd);
    kx[(size_t)t * H * (d + rd) + i] = j < d ? kn[((size_t)t * H + h) * d + j] : shared_part[j - d];
  }
}

// out[t][h * out_hs + n] = sum_k a[t][h * a_hs + k] * w[h][n][k], float32 sums; a: float32 rows of lda floats, out: rows of ldo values.
// Tiles of 32 tokens x TN columns (TN 64, or 16 when the step has few tokens: four times the blocks), K in steps of 32.
constexpr int HM_TT = 32, HM_KC = 32;
template <typename TW, typename TO, int TN>
__global__ void __launch_bounds__(256)
head_matmul_kernel(const float* __restrict__ a, int lda, int a_hs, const TW* __restrict__ w, TO* __restrict__ out, int ldo,
                   int out_hs, int n_tokens, int K, int N) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NJ = TN / 16;      // columns a thread
  __shared__ float As[HM_TT][HM_KC + 1];
  __shared__ float Ws[TN][HM_KC + 1];
  const int h = blockIdx.z, t0 = blockIdx.x * HM_TT, n0 = blockIdx.y * TN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;     // 16 column groups, 16 row groups of 2
  const TW* wh = w + (size_t)h * N * K;
  float acc[2][NJ] = {};
  for (int k0 = 0; k0 < K; k0 += HM_KC) {
    for (int i = threadIdx.x; i < HM_TT * HM_KC; i += 256) {
      const int r = i / HM_KC, k = i - r * HM_KC;
      As[r][k] = (t0 + r < n_tokens && k0 + k < K) ? a[(size_t)(t0 + r) * lda + (size_t)h * a_hs + k0 + k] : 0.f;
    }
    for (int i = threadIdx.x; i < TN * HM_KC; i += 256) {
      const int r = i / HM_KC, k = i - r * HM_KC;
      Ws[r][k] = (n0 + r < N && k0 + k < K) ? to_f32(wh[(size_t)(n0 + r) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < HM_KC; ++k) {
      const float a0 = As[ty * 2][k], a1 = As[ty * 2 + 1][k];
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const float wv = Ws[tx + 16 * j][k];
        acc[0][j] = fmaf(a0, wv, acc[0][j]);
        acc[1][j] = fmaf(a1, wv, acc[1][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int t = t0 + ty * 2 + i, n = n0 + tx + 16 * j;
      if (t < n_tokens && n < N) out[(size_t)t * ldo + (size_t)h * out_hs + n] = from_f32<TO>(acc[i][j]);
    }
}

// x[t][:] += b[:]
__global__ void add_row_bias_kernel(float* __restrict__ x, const float* __restrict__ b, int dim) {
  pdl_launch_dependents();
  pdl_wait();
  float* row = x + (size_t)blockIdx.x * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) row[i] += b[i];
}

// q . k over n dimensions, q float32 in shared memory; four running sums
__device__ __forceinline__ float ma_dot(const float* __restrict__ q, const float* __restrict__ k, int n, bool vec) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int i = 0;
  if (vec)
    for (; i + 4 <= n; i += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(k + i);
      const float4 qv = *reinterpret_cast<const float4*>(q + i);
      a0 = fmaf(qv.x, kv.x, a0); a1 = fmaf(qv.y, kv.y, a1); a2 = fmaf(qv.z, kv.z, a2); a3 = fmaf(qv.w, kv.w, a3);
    }
  for (; i < n; ++i) a0 = fmaf(q[i], k[i], a0);
  return (a0 + a1) + (a2 + a3);
}
__device__ __forceinline__ float ma_dot(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int n, bool vec) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int i = 0;
  if (vec)
    for (; i + 8 <= n; i += 8) {
      const uint4 kv = *reinterpret_cast<const uint4*>(k + i);
      const float4 q0 = *reinterpret_cast<const float4*>(q + i), q1 = *reinterpret_cast<const float4*>(q + i + 4);
      a0 = fmaf(q0.x, __uint_as_float(kv.x << 16), a0); a1 = fmaf(q0.y, __uint_as_float(kv.x & 0xffff0000u), a1);
      a2 = fmaf(q0.z, __uint_as_float(kv.y << 16), a2); a3 = fmaf(q0.w, __uint_as_float(kv.y & 0xffff0000u), a3);
      a0 = fmaf(q1.x, __uint_as_float(kv.z << 16), a0); a1 = fmaf(q1.y, __uint_as_float(kv.z & 0xffff0000u), a1);
      a2 = fmaf(q1.z, __uint_as_float(kv.w << 16), a2); a3 = fmaf(q1.w, __uint_as_float(kv.w & 0xffff0000u), a3);
    }
  for (; i < n; ++i) a0 = fmaf(q[i], __bfloat162float(k[i]), a0);
  return (a0 + a1) + (a2 + a3);
}

constexpr int MA_MAX_WARPS = 8;

// A block per (token, query head); its warps take the visible keys in turns of 32 (a lane a key), each with its own
// running maximum, denominator and weighted values, merged at the end through shared memory in a fixed order.
// Dynamic shared memory: the scaled query (dk floats), then per warp its maximum, its denominator and dv values.
// DVR: value dimensions a lane holds (d = lane + 32 r), so value heads of up to 32 DVR dimensions.
template <typename T, typename TO, int DVR>
__global__ void __launch_bounds__(MA_MAX_WARPS * 32)
masked_attn_kernel(const float* __restrict__ q, TO* __restrict__ out, const T* __restrict__ kcache, const T* __restrict__ vbase, int ldv,
                   const int32_t* __restrict__ tok_pos, const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ page_table,
                   int table_stride, int n_pages, int H, int G, int dk, int dv, float scale, int mask, int mask_size,
                   const float* __restrict__ sink, int vec_k, int maps, const float* __restrict__ gate, int ldg, int n_splits,
                   float* __restrict__ part) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float ma_smem[];
  const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, NW = blockDim.x >> 5;
  const int dkp = (dk + 3) & ~3;
  float* qh = ma_smem;
  float* wm = ma_smem + dkp;
  float* wl = wm + NW;
  float* wo = wl + NW;             // [NW][dv]
  const int pos = tok_pos[t];
  if (pos < 0) return;
  // `maps` > 1: a head is `maps` runs of dk dimensions side by side, in the queries and in a key row; each run is an
  // attention of its own over the head's values.  blockIdx.y = head * maps + run.
  const int HV = H * maps, kp = dk * maps, koff = (h % maps) * dk;
  const int g = (h / maps) / (H / G);
  const int32_t* table = page_table + (size_t)tok_seq[t] * table_stride;
  const float* qrow = q + ((size_t)t * HV + h) * dk;
  for (int i = threadIdx.x; i < dk; i += blockDim.x) qh[i] = qrow[i] * scale;
  __syncthreads();
  const int lo = first_key(pos, mask, mask_size), n_keys = pos - lo + 1;
  const int n_chunks = (n_keys + 31) >> 5;
  float m = -INFINITY, l = 0.f;
  float o[DVR];
#pragma unroll
  for (int r = 0; r < DVR; ++r) o[r] = 0.f;
  // `n_splits` > 1: the token's chunks of 32 keys are dealt to so many blocks (blockIdx.z), each of which leaves its maximum,
  // denominator and weighted values for the fold kernel (the sink and the gate join there)
  const int per_split = (n_chunks + n_splits - 1) / n_splits;
  const int c_end = min(n_chunks, ((int)blockIdx.z + 1) * per_split);
  for (int c = blockIdx.z * per_split + warp; c < c_end; c += NW) {
    const int n_here = min(32, n_keys - c * 32);
    float sc = -INFINITY;
    int vrow = -1;
    if (lane < n_here) {
      const int p = lo + c * 32 + lane;
      const int page = table[p / PAGE];
      if (page >= 0 && page < n_pages) {
        vrow = (page * G + g) * PAGE + p % PAGE;
        sc = ma_dot(qh, kcache + (size_t)vrow * kp + koff, dk, vec_k != 0);
      }
    }
    const float m_new = fmaxf(m, warp_max(sc));
    if (m_new == -INFINITY) continue;
    const float w = sc == -INFINITY ? 0.f : expf(sc - m_new);
    const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(w);
    m = m_new;
#pragma unroll
    for (int r = 0; r < DVR; ++r) o[r] *= corr;
    // the values of VB keys are requested before the first is used: with one key's loads at a time a chunk of 32 keys was 32
    // trips to memory one after the other (8 sequences x 32 heads over 2,048 keys: 105 -> 84 us a layer in a launch list)
    constexpr int VB = DVR <= 2 ? 16 : (DVR <= 4 ? 8 : 4);
    for (int j0 = 0; j0 < n_here; j0 += VB) {
      float wv[VB];
      T vals[VB][DVR];
#pragma unroll
      for (int x = 0; x < VB; ++x) {
        const int j = min(j0 + x, 31);
        const float wj = __shfl_sync(0xffffffffu, w, j);
        const int vr_i = __shfl_sync(0xffffffffu, vrow, j);
        wv[x] = j0 + x < n_here && vr_i >= 0 ? wj : 0.f;
        const T* vr = vbase + (size_t)max(vr_i, 0) * ldv;
#pragma unroll
        for (int r = 0; r < DVR; ++r) {
          const int d = lane + 32 * r;
          vals[x][r] = d < dv && wv[x] != 0.f ? vr[d] : from_f32<T>(0.f);
        }
      }
#pragma unroll
      for (int x = 0; x < VB; ++x)
#pragma unroll
        for (int r = 0; r < DVR; ++r) o[r] = fmaf(wv[x], to_f32(vals[x][r]), o[r]);
    }
  }
  if (lane == 0) { wm[warp] = m; wl[warp] = l; }
#pragma unroll
  for (int r = 0; r < DVR; ++r) {
    const int d = lane + 32 * r;
    if (d < dv) wo[warp * dv + d] = o[r];
  }
  __syncthreads();
  if (n_splits > 1) {
    float M = -INFINITY, L = 0.f;
    for (int w2 = 0; w2 < NW; ++w2) M = fmaxf(M, wm[w2]);
    for (int w2 = 0; w2 < NW; ++w2) L += wm[w2] == -INFINITY ? 0.f : wl[w2] * expf(wm[w2] - M);
    float* dst = part + (((size_t)t * HV + h) * n_splits + blockIdx.z) * (2 + dv);
    if (threadIdx.x == 0) { dst[0] = M; dst[1] = L; }
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
      float acc = 0.f;
      for (int w2 = 0; w2 < NW; ++w2)
        if (wm[w2] != -INFINITY) acc = fmaf(wo[w2 * dv + d], expf(wm[w2] - M), acc);
      dst[2 + d] = acc;
    }
    return;
  }
  float M = sink ? sink[h / maps] : -INFINITY;
  for (int w2 = 0; w2 < NW; ++w2) M = fmaxf(M, wm[w2]);
  float L = sink ? expf(sink[h / maps] - M) : 0.f;
  for (int w2 = 0; w2 < NW; ++w2) L += wm[w2] == -INFINITY ? 0.f : wl[w2] * expf(wm[w2] - M);
  float inv = L > 0.f ? 1.0f / L : 0.f;
  if (gate) inv *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h / maps]));      // the head's output gate: sigmoid of its logit
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float acc = 0.f;
    for (int w2 = 0; w2 < NW; ++w2)
      if (wm[w2] != -INFINITY) acc = fmaf(wo[w2 * dv + d], expf(wm[w2] - M), acc);
    out[((size_t)t * HV + h) * dv + d] = from_f32<TO>(acc * inv);
  }
}

// ---- prompt steps
// A block = up to 32 (token, query head) rows of one key/value head and of one run of consecutive tokens (a tile of the
// step's metadata); a page of 64 keys with their values is staged in shared memory as float32 once for all the rows.
// A warp owns four rows, so a key element read from shared memory serves four multiply-adds; lanes own keys for the
// scores and value dimensions for the weighted sum.  Row r sees key p iff first[r] <= p <= its own position.
constexpr int TM_RW = 4, TM_WARPS = 8, TM_ROWS = TM_RW * TM_WARPS, TM_KEYS = PAGE;

// PAGE rows of n values from global memory (row pitch `src_pitch`) into shared memory as float32 (row pitch `dst_pitch`); rows from
// `valid` on become zeros.  16 bytes a load where the rows allow it: a thread then has a few loads in flight instead of
// one per value.
template <typename T>
__device__ __forceinline__ void stage_rows(float* __restrict__ dst, int dst_pitch, const T* __restrict__ src, int src_pitch, int n, int valid) {
  constexpr int V = 16 / (int)sizeof(T);
  const bool vec = n % V == 0 && src_pitch % V == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  if (vec) {
    const int per_row = n / V;
#pragma unroll 4
    for (int i = threadIdx.x; i < PAGE * per_row; i += blockDim.x) {
      const int j = i / per_row, d = (i - j * per_row) * V;
      float* o = dst + j * dst_pitch + d;
      if (j < valid) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + (size_t)j * src_pitch + d);
        if constexpr (sizeof(T) == 4) {
          o[0] = __uint_as_float(raw.x); o[1] = __uint_as_float(raw.y); o[2] = __uint_as_float(raw.z); o[3] = __uint_as_float(raw.w);
        } else {
          o[0] = __uint_as_float(raw.x << 16); o[1] = __uint_as_float(raw.x & 0xffff0000u);
          o[2] = __uint_as_float(raw.y << 16); o[3] = __uint_as_float(raw.y & 0xffff0000u);
          o[4] = __uint_as_float(raw.z << 16); o[5] = __uint_as_float(raw.z & 0xffff0000u);
          o[6] = __uint_as_float(raw.w << 16); o[7] = __uint_as_float(raw.w & 0xffff0000u);
        }
      } else {
#pragma unroll
        for (int q = 0; q < V; ++q) o[q] = 0.f;
      }
    }
  } else {
    for (int i = threadIdx.x; i < PAGE * n; i += blockDim.x) {
      const int j = i / n, d = i - j * n;
      dst[j * dst_pitch + d] = j < valid ? to_f32(src[(size_t)j * src_pitch + d]) : 0.f;
    }
  }
}

template <typename T, typename TO, int NC>    // NC = ceil(dv / 32): value dimensions a lane owns
__global__ void __launch_bounds__(TM_WARPS * 32)
masked_attn_tiled_kernel(const float* __restrict__ q, TO* __restrict__ out, const T* __restrict__ kcache, const T* __restrict__ vcache,
                         const int32_t* __restrict__ page_table, int table_stride, int n_pages, const int32_t* __restrict__ tile_seq,
                         const int32_t* __restrict__ tile_tok0, const int32_t* __restrict__ tile_ntok, const int32_t* __restrict__ tile_pos0,
                         int H, int G, int dk, int dv, float scale, int mask, int mask_size, const float* __restrict__ sink,
                         int n_splits, float* __restrict__ part, int maps, const float* __restrict__ gate, int ldg) {
  extern __shared__ float tm_smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int ks = dk + 1;                        // padded key row: lanes read different rows
  const bool own_v = vcache != nullptr;
  const int vs = own_v ? dv : ks;               // a staged value row's pitch (values inside the keys: the key's)
  float* Ks = tm_smem;                          // [TM_KEYS][dk + 1]
  float* Vs = own_v ? Ks + TM_KEYS * ks : Ks;   // [TM_KEYS][dv]
  float* Qs = Ks + TM_KEYS * ks + (own_v ? TM_KEYS * dv : 0);   // [TM_ROWS][dk]
  float* Ps = Qs + TM_ROWS * dk;                // [TM_ROWS][TM_KEYS]
  // `maps` > 1: a head is `maps` runs of dk dimensions side by side (queries and key rows); blockIdx.y = kv head * maps + run,
  // and the block's rows are the run's queries of the heads that share the kv head.  Row (token, head, run) of q and out.
  const int tile = blockIdx.x, g = blockIdx.y / maps, mp = blockIdx.y % maps, grp = H / G, HV = H * maps, kfull = dk * maps;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int seq = tile_seq[tile], tok0 = tile_tok0[tile], ntok = tile_ntok[tile], pos0 = tile_pos0[tile];
  // `page_table` null: the keys and values are the step's own rows [token][kv_head][dk or dv] (every sequence of the step
  // starts at position 0, so position p of the tile's sequence is packed row tok0 - pos0 + p)
  const bool paged = page_table != nullptr;
  const int32_t* pages = paged ? page_table + (size_t)seq * table_stride : nullptr;
  const int k_pitch = paged ? kfull : G * kfull, v_pitch = paged ? dv : G * dv;
  // n_splits > 1: the pages a tile's rows see are dealt to n_splits blocks (blockIdx.z = row tile * n_splits + split); each
  // leaves its rows' maximum, denominator and weighted values in `part` [token][head][split][2 + dv] and `masked_attn_fold`
  // merges them: steps of one token a sequence whose query heads share few key heads
  const int split = blockIdx.z % n_splits;
  const int rows_total = ntok * grp, row_base = (blockIdx.z / n_splits) * TM_ROWS;
  if (row_base >= rows_total) return;
  const int rows_here = min(TM_ROWS, rows_total - row_base);
  const int last_pos = pos0 + (row_base + rows_here - 1) / grp, first_pos = pos0 + row_base / grp;
  for (int i = threadIdx.x; i < TM_ROWS * dk; i += blockDim.x) {
    const int r = i / dk, d = i - r * dk;
    const int rr = row_base + r, tok = rr / grp, head = g * grp + rr % grp;
    Qs[i] = r < rows_here ? q[((size_t)(tok0 + tok) * HV + head * maps + mp) * dk + d] : 0.f;
  }
  float m[TM_RW], l[TM_RW], acc[TM_RW][NC];
  int limit[TM_RW], first[TM_RW];
#pragma unroll
  for (int r = 0; r < TM_RW; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
    const int rr = row_base + warp * TM_RW + r;
    limit[r] = rr < rows_total ? pos0 + rr / grp : -1;                       // the row's own position; -1: no row
    first[r] = limit[r] < 0 ? 0 : first_key(limit[r], mask, mask_size);
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;
  }
  int kt_begin = first_key(first_pos, mask, mask_size) / PAGE, kt_end = last_pos / PAGE;
  if (n_splits > 1) {
    const int per = (kt_end - kt_begin + n_splits) / n_splits;
    kt_begin += split * per;
    kt_end = min(kt_end, kt_begin + per - 1);
  }
  for (int kt = kt_begin; kt <= kt_end; ++kt) {
    const int page = paged ? pages[kt] : 0;
    const bool held = !paged || (page >= 0 && page < n_pages);
    const size_t first_row = paged ? ((size_t)(held ? page : 0) * G + g) * PAGE : ((size_t)(tok0 - pos0 + kt * PAGE) * G + g);
    const T* kp = kcache + first_row * kfull + mp * dk;
    const int valid = held ? min(PAGE, last_pos + 1 - kt * PAGE) : 0;   // rows of the page that hold this block's keys
    __syncthreads();
    stage_rows<T>(Ks, ks, kp, k_pitch, dk, valid);      // what lies behind `valid` is not this sequence's: never let it in
    if (own_v) stage_rows<T>(Vs, dv, vcache + first_row * dv, v_pitch, dv, valid);
    __syncthreads();
    const int base = kt * PAGE;
    int any_hi = -1, any_lo = 0x7fffffff;
#pragma unroll
    for (int r = 0; r < TM_RW; ++r)
      if (limit[r] >= first[r]) { any_hi = max(any_hi, limit[r]); any_lo = min(any_lo, first[r]); }
    if (base > any_hi || base + TM_KEYS - 1 < any_lo) continue;     // none of this warp's rows sees any of these keys
    const int i0 = base + lane, i1 = i0 + 32;
    float s0[TM_RW] = {}, s1[TM_RW] = {};
    const float* k0 = Ks + lane * ks;
    const float* k1 = Ks + (lane + 32) * ks;
    const float* qw = Qs + warp * TM_RW * dk;
    for (int d = 0; d < dk; ++d) {
      const float a = k0[d], b = k1[d];
#pragma unroll
      for (int r = 0; r < TM_RW; ++r) {
        const float qv = qw[r * dk + d];
        s0[r] = fmaf(qv, a, s0[r]);
        s1[r] = fmaf(qv, b, s1[r]);
      }
    }
    float corr[TM_RW];
#pragma unroll
    for (int r = 0; r < TM_RW; ++r) {
      const float a = i0 >= first[r] && i0 <= limit[r] ? s0[r] * scale : -INFINITY;
      const float b = i1 >= first[r] && i1 <= limit[r] ? s1[r] * scale : -INFINITY;
      const float mx = fmaxf(m[r], warp_max(fmaxf(a, b)));
      float p0 = 0.f, p1 = 0.f;
      corr[r] = 1.f;
      if (mx != -INFINITY) {      // uniform over the warp
        corr[r] = expf(m[r] - mx);
        p0 = expf(a - mx);
        p1 = expf(b - mx);
        l[r] = l[r] * corr[r] + warp_sum(p0 + p1);
        m[r] = mx;
      }
      Ps[(warp * TM_RW + r) * TM_KEYS + lane] = p0;
      Ps[(warp * TM_RW + r) * TM_KEYS + lane + 32] = p1;
    }
    __syncwarp();
#pragma unroll
    for (int r = 0; r < TM_RW; ++r)
#pragma unroll
      for (int c = 0; c < NC; ++c) acc[r][c] *= corr[r];
    const float* pw = Ps + warp * TM_RW * TM_KEYS;
    for (int j = 0; j < valid; ++j) {
      float v[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int d = lane + 32 * c;
        v[c] = d < dv ? Vs[j * vs + d] : 0.f;
      }
#pragma unroll
      for (int r = 0; r < TM_RW; ++r) {
        const float pj = pw[r * TM_KEYS + j];
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[r][c] = fmaf(pj, v[c], acc[r][c]);
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int r = 0; r < TM_RW; ++r) {
    const int rr = row_base + warp * TM_RW + r;
    if (rr >= rows_total) continue;
    const int tok = rr / grp, head = g * grp + rr % grp;
    if (n_splits > 1) {
      float* dst = part + (((size_t)(tok0 + tok) * HV + head * maps + mp) * n_splits + split) * (2 + dv);
      if (lane == 0) { dst[0] = m[r]; dst[1] = l[r]; }
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int d = lane + 32 * c;
        if (d < dv) dst[2 + d] = acc[r][c];
      }
      continue;
    }
    float lr = l[r], fix = 1.f;
    if (sink) {                                   // the sink: one more term of the denominator, no value
      const float sk = sink[head], mx = fmaxf(m[r], sk);
      fix = m[r] == -INFINITY ? 0.f : expf(m[r] - mx);
      lr = lr * fix + expf(sk - mx);
    }
    float inv = lr > 0.f ? fix / lr : 0.f;
    if (gate) inv *= 1.0f / (1.0f + expf(-gate[(size_t)(tok0 + tok) * ldg + head]));      // the head's output gate
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int d = lane + 32 * c;
      if (d < dv) out[((size_t)(tok0 + tok) * HV + head * maps + mp) * dv + d] = from_f32<TO>(acc[r][c] * inv);
    }
  }
}

// out[t][h][:] from the splits' partial results [t][h][split][2 + dv]: maxima, denominators, weighted values; the sink joins here
template <typename TO>
__global__ void masked_attn_fold_kernel(const float* __restrict__ part, TO* __restrict__ out, const float* __restrict__ sink, int H, int dv,
                                        int n_splits, const float* __restrict__ gate, int ldg, int maps) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const float* p = part + ((size_t)t * H + h) * n_splits * (2 + dv);
  float M = sink ? sink[h] : -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, p[(size_t)s * (2 + dv)]);
  float L = sink ? expf(sink[h] - M) : 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = p[(size_t)s * (2 + dv)];
    if (ms != -INFINITY) L += p[(size_t)s * (2 + dv) + 1] * expf(ms - M);
  }
  float inv = L > 0.f ? 1.0f / L : 0.f;
  if (gate) inv *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h / maps]));      // the head's output gate
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = p[(size_t)s * (2 + dv)];
      if (ms != -INFINITY) acc = fmaf(p[(size_t)s * (2 + dv) + 2 + d], expf(ms - M), acc);
    }
    out[((size_t)t * H + h) * dv + d] = from_f32<TO>(acc * inv);
  }
}

// Two attention maps of a head into one ("differential" attention): a [tokens][H][2][dv] float32;
// o = a_1 - lambda a_2, then o / sqrt(mean(o^2) + eps) over the head's dv values, times `post` (and `w` [dv], if given).
// A warp per (token, head).
template <typename TO>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const float* __restrict__ a, TO* __restrict__ out, float lambda, float eps, float post, const float* __restrict__ w,
                    int n_rows, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const float* a1 = a + (size_t)row * 2 * dv;
  const float* a2 = a1 + dv;
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) {
    const float o = a1[d] - lambda * a2[d];
    ss = fmaf(o, o, ss);
  }
  const float inv = post / sqrtf(warp_sum(ss) / (float)dv + eps);
  for (int d = lane; d < dv; d += 32) {
    const float o = a1[d] - lambda * a2[d];
    out[(size_t)row * dv + d] = from_f32<TO>(o * inv * (w ? w[d] : 1.0f));
  }
}

}  // namespace edgelm

using namespace edgelm;

extern "C" int edgelm_diff_combine(const float* a, void* out, int out_dtype, float lambda, float eps, float post, const float* w, int n_rows,
                                   int dv, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  EL_REFUSE(n_rows > 0 && dv >= 1, "diff_combine: bad sizes");
  const dim3 grid((n_rows + 3) / 4), block(128);
  const int bit = pdl_bit_for_tokens(n_rows);
  if (out_dtype == DT_F32) launch_pdl(bit, diff_combine_kernel<float>, grid, block, (size_t)0, stream, a, (float*)out, lambda, eps, post, w, n_rows, dv);
  else if (out_dtype == DT_BF16) launch_pdl(bit, diff_combine_kernel<__nv_bfloat16>, grid, block, (size_t)0, stream, a, (__nv_bfloat16*)out, lambda, eps, post, w, n_rows, dv);
  else EL_REFUSE(false, "diff_combine: unknown dtype code %d", out_dtype);
  EL_LAUNCH_CHECK("diff_combine");
  return 0;
}

extern "C" int edgelm_rotate_append(const float* qkv, const float* bias, float* q_out, const int32_t* tok_pos, const int32_t* tok_seq,
                                    const int32_t* page_table, int table_stride, int n_pages, void* kcache, void* vcache, int dtype,
                                    int n_tokens, int H, int G, int dk, int dv, int rot, int interleaved, const double* freq, int* err,
                                    int maps, const float* q_norm, const float* k_norm, float eps, int ldq, const float* conv_w, int taps,
                                    float* conv_state, const int32_t* seq_tok0, const int32_t* seq_slot, int move_tail, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(conv_w == nullptr || (taps >= 1 && seq_tok0 != nullptr && seq_slot != nullptr && (taps == 1 || conv_state != nullptr)),
            "rotate_append: a filter of %d taps needs the sequences' first rows, their slots and the tails", taps);
  ConvAhead conv;
  conv.w = conv_w; conv.state = conv_state; conv.seq_tok0 = seq_tok0; conv.seq_slot = seq_slot; conv.taps = taps; conv.move_tail = move_tail;
  if (ldq == 0) ldq = (H + G) * dk + G * dv;
  EL_REFUSE(ldq >= (H + G) * dk + G * dv, "rotate_append: rows of %d values do not hold the heads", ldq);
  EL_REFUSE(maps >= 1 && dk % maps == 0 && rot <= dk / maps, "rotate_append: %d maps of a head of %d with %d rotated dimensions", maps, dk, rot);
  EL_REFUSE(n_tokens > 0 && H > 0 && G > 0 && H % G == 0, "rotate_append: %d query heads over %d key/value heads", H, G);
  EL_REFUSE(dk >= 1 && dk <= 2048 && dv >= 1, "rotate_append: head sizes %d / %d are not taken", dk, dv);
  EL_REFUSE(rot >= 0 && rot <= dk && rot % 2 == 0 && (rot == 0 || freq != nullptr), "rotate_append: %d rotated dimensions of %d", rot, dk);
  const size_t smem = (size_t)MA_WARPS * dk * sizeof(float);
  const dim3 grid(n_tokens, (H + G + MA_WARPS - 1) / MA_WARPS), block(MA_WARPS * 32);
  const int bit = pdl_bit_for_tokens(n_tokens);
  if (dtype == DT_F32)
    launch_pdl(bit, rotate_append_kernel<float>, grid, block, smem, stream, qkv, bias, q_out, tok_pos, tok_seq, page_table, table_stride,
               n_pages, (float*)kcache, (float*)vcache, H, G, dk, dv, rot, interleaved, freq, err, maps, q_norm, k_norm, eps, ldq, conv);
  else if (dtype == DT_BF16)
    launch_pdl(bit, rotate_append_kernel<__nv_bfloat16>, grid, block, smem, stream, qkv, bias, q_out, tok_pos, tok_seq, page_table,
               table_stride, n_pages, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, H, G, dk, dv, rot, interleaved, freq, err, maps, q_norm, k_norm, eps, ldq, conv);
  else
    EL_REFUSE(false, "rotate_append: unknown dtype code %d", dtype);
  EL_LAUNCH_CHECK("rotate_append");
  return 0;
}

extern "C" int edgelm_latent_prepare(const float* u, int ldu, int kv_off, int has_kv, float* q_out, int q_pitch, int q_off, int copy_q,
                                     const float* norm_w, float eps, const int32_t* tok_pos, const int32_t* tok_seq,
                                     const int32_t* page_table, int table_stride, int n_pages, void* kcache, void* row_out, int dtype,
                                     int n_tokens, int H, int d, int rd, int r, const double* freq, int* err, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && H > 0 && d >= 0 && r >= 1 && rd >= 0 && rd % 2 == 0, "latent_prepare: sizes heads %d, %d + %d, latent %d", H, d, rd, r);
  EL_REFUSE(rd == 0 || freq != nullptr, "latent_prepare: no frequencies");
  EL_REFUSE(H * (d + rd) <= ldu && (!has_kv || kv_off + r + rd <= ldu), "latent_prepare: rows of %d values are too short", ldu);
  EL_REFUSE(q_off >= (copy_q ? d : 0) && q_off + rd <= q_pitch, "latent_prepare: a query head of %d values does not hold %d at %d", q_pitch, rd, q_off);
  const int bit = pdl_bit_for_tokens(n_tokens);
  if (dtype == DT_F32)
    launch_pdl(bit, latent_prepare_kernel<float>, dim3(n_tokens), dim3(256), (size_t)0, stream, u, ldu, kv_off, has_kv, q_out, q_pitch, q_off, copy_q,
               norm_w, eps, tok_pos, tok_seq, page_table, table_stride, n_pages, (float*)kcache, (float*)row_out, H, d, rd, r, freq, err);
  else if (dtype == DT_BF16)
    launch_pdl(bit, latent_prepare_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), (size_t)0, stream, u, ldu, kv_off, has_kv, q_out, q_pitch, q_off,
               copy_q, norm_w, eps, tok_pos, tok_seq, page_table, table_stride, n_pages, (__nv_bfloat16*)kcache, (__nv_bfloat16*)row_out, H, d, rd,
               r, freq, err);
  else
    EL_REFUSE(false, "latent_prepare: unknown dtype code %d", dtype);
  EL_LAUNCH_CHECK("latent_prepare");
  return 0;
}

extern "C" int edgelm_latent_expand_keys(const void* kn, const void* rows, void* kx, int dtype, int n_tokens, int H, int d, int rd, int r,
                                         cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && H > 0 && d >= 0 && rd >= 0 && d + rd >= 1 && r >= 1, "latent_expand_keys: bad sizes");
  if (dtype == DT_F32)
    launch_pdl(0, latent_expand_keys_kernel<float>, dim3(n_tokens), dim3(256), (size_t)0, stream, (const float*)kn, (const float*)rows, (float*)kx, H, d, rd, r);
  else if (dtype == DT_BF16)
    launch_pdl(0, latent_expand_keys_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), (size_t)0, stream, (const __nv_bfloat16*)kn,
               (const __nv_bfloat16*)rows, (__nv_bfloat16*)kx, H, d, rd, r);
  else
    EL_REFUSE(false, "latent_expand_keys: unknown dtype code %d", dtype);
  EL_LAUNCH_CHECK("latent_expand_keys");
  return 0;
}

extern "C" int edgelm_head_matmul(const float* a, int lda, int a_hs, const void* w, int w_dtype, void* out, int out_dtype, int ldo, int out_hs,
                                  int n_tokens, int H, int K, int N, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && H > 0 && K > 0 && N > 0 && H <= 65535, "head_matmul: bad sizes heads %d, K %d, N %d", H, K, N);
  const int tn = n_tokens <= 64 ? 16 : 64;
  const dim3 grid((n_tokens + HM_TT - 1) / HM_TT, (N + tn - 1) / tn, H), block(256);
  const int bit = pdl_bit_for_tokens(n_tokens);
#define EL_HM(TW, TO) do { if (tn == 16) launch_pdl(bit, head_matmul_kernel<TW, TO, 16>, grid, block, (size_t)0, stream, a, lda, a_hs, (const TW*)w, (TO*)out, ldo, out_hs, n_tokens, K, N); \
    else launch_pdl(bit, head_matmul_kernel<TW, TO, 64>, grid, block, (size_t)0, stream, a, lda, a_hs, (const TW*)w, (TO*)out, ldo, out_hs, n_tokens, K, N); } while (0)
  if (w_dtype == DT_F32 && out_dtype == DT_F32) EL_HM(float, float);
  else if (w_dtype == DT_BF16 && out_dtype == DT_F32) EL_HM(__nv_bfloat16, float);
  else if (w_dtype == DT_BF16 && out_dtype == DT_BF16) EL_HM(__nv_bfloat16, __nv_bfloat16);
  else EL_REFUSE(false, "head_matmul: dtype codes %d -> %d are not taken", w_dtype, out_dtype);
#undef EL_HM
  EL_LAUNCH_CHECK("head_matmul");
  return 0;
}

extern "C" int edgelm_add_row_bias(float* x, const float* b, int n_tokens, int dim, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && dim > 0, "add_row_bias: bad sizes");
  launch_pdl(pdl_bit_for_tokens(n_tokens), add_row_bias_kernel, dim3(n_tokens), dim3(dim >= 1024 ? 256 : 128), (size_t)0, stream, x, b, dim);
  EL_LAUNCH_CHECK("add_row_bias");
  return 0;
}

static int masked_common_check(const char* what, int H, int G, int dk, int dv, int mask, int mask_size, int dtype, int out_dtype) {
  EL_REFUSE(H > 0 && G > 0 && H % G == 0, "%s: %d query heads over %d key/value heads", what, H, G);
  EL_REFUSE(dk >= 1 && dk <= 1024 && dv >= 1 && dv <= 512, "%s: head sizes %d / %d are not taken (keys to 1024, values to 512)", what, dk, dv);
  EL_REFUSE(mask == MASK_CAUSAL || ((mask == MASK_WINDOW || mask == MASK_CHUNK) && mask_size >= 1), "%s: mask %d of size %d", what, mask, mask_size);
  EL_REFUSE((dtype == DT_F32 && out_dtype == DT_F32) || (dtype == DT_BF16 && (out_dtype == DT_F32 || out_dtype == DT_BF16)),
            "%s: dtype codes %d -> %d are not taken", what, dtype, out_dtype);
  return 0;
}

template <typename T, typename TO, int DVR>
static void launch_masked(const float* q, void* out, const void* kcache, const void* vcache, const int32_t* tok_pos, const int32_t* tok_seq,
                          const int32_t* page_table, int table_stride, int n_pages, int n_tokens, int H, int G, int dk, int dv, float scale,
                          int mask, int mask_size, const float* sink, int warps, int maps, const float* gate, int ldg, int n_splits, float* part,
                          cudaStream_t stream) {
  const T* vb = vcache ? (const T*)vcache : (const T*)kcache;
  const int ldv = vcache ? dv : dk;
  const int vec_k = (dk % (16 / (int)sizeof(T)) == 0) && ((uintptr_t)kcache % 16 == 0);
  const size_t smem = ((size_t)((dk + 3) & ~3) + (size_t)warps * (2 + dv)) * sizeof(float);
  auto kern = masked_attn_kernel<T, TO, DVR>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_pdl(pdl_bit_for_tokens(n_tokens), kern, dim3(n_tokens, H * maps, n_splits), dim3(warps * 32), smem, stream, q, (TO*)out, (const T*)kcache, vb, ldv,
             tok_pos, tok_seq, page_table, table_stride, n_pages, H, G, dk, dv, scale, mask, mask_size, sink, vec_k, maps, gate, ldg, n_splits, part);
  if (n_splits > 1 && cudaPeekAtLastError() == cudaSuccess)
    launch_pdl(pdl_bit_for_tokens(n_tokens), masked_attn_fold_kernel<TO>, dim3(n_tokens, H * maps), dim3(dv >= 256 ? 256 : 128), (size_t)0, stream,
               (const float*)part, (TO*)out, sink, H * maps, dv, n_splits, gate, ldg, maps);
}

// `vcache` null: the values are the first dv dimensions of the key rows.  `max_keys`: the most keys a token of the step sees
// (chooses how many warps share a token's keys).  `n_splits` > 1: a token's keys are dealt to so many blocks, whose partial
// results go through `part` (n_tokens H maps n_splits (2 + dv) floats) and are merged by a second launch.  `maps` > 1: every query head and key row holds `maps` runs of dk dimensions,
// each an attention of its own over the head's values; q [tokens][H][maps][dk], out [tokens][H][maps][dv].
extern "C" int edgelm_masked_attn(const float* q, void* out, int out_dtype, const void* kcache, const void* vcache, int dtype,
                                  const int32_t* tok_pos, const int32_t* tok_seq, const int32_t* page_table, int table_stride, int n_pages,
                                  int n_tokens, int H, int G, int dk, int dv, float scale, int mask, int mask_size, const float* sink,
                                  int max_keys, int maps, const float* gate, int ldg, int n_splits, float* part, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_splits >= 1 && n_splits <= 64 && (n_splits == 1 || part != nullptr), "masked_attn: %d splits", n_splits);
  if (n_splits > 1) max_keys = (max_keys + n_splits - 1) / n_splits;
  if (masked_common_check("masked_attn", H, G, dk, dv, mask, mask_size, dtype, out_dtype)) return -1;
  EL_REFUSE(maps >= 1 && H * maps <= 65535 && (maps == 1 || (sink == nullptr && vcache != nullptr)), "masked_attn: %d maps take no sink and values of their own", maps);
  EL_REFUSE(vcache != nullptr || dv <= dk, "masked_attn: values of %d inside keys of %d", dv, dk);
  const int warps = max_keys <= 64 ? 2 : (max_keys <= 256 ? 4 : MA_MAX_WARPS);
#define EL_MA2(T, TO, DVR) launch_masked<T, TO, DVR>(q, out, kcache, vcache, tok_pos, tok_seq, page_table, table_stride, n_pages, n_tokens, H, G, dk, dv, scale, mask, mask_size, sink, warps, maps, gate, ldg, n_splits, part, stream)
#define EL_MA(DVR) do { if (dtype == DT_F32) EL_MA2(float, float, DVR); else if (out_dtype == DT_F32) EL_MA2(__nv_bfloat16, float, DVR); else EL_MA2(__nv_bfloat16, __nv_bfloat16, DVR); } while (0)
  if (dv <= 32) EL_MA(1); else if (dv <= 64) EL_MA(2); else if (dv <= 128) EL_MA(4); else if (dv <= 256) EL_MA(8); else EL_MA(16);
#undef EL_MA
#undef EL_MA2
  EL_LAUNCH_CHECK("masked_attn");
  return 0;
}

template <typename T, typename TO, int NC>
static int launch_masked_tiled(const float* q, void* out, const void* kcache, const void* vcache, const int32_t* page_table, int table_stride,
                               int n_pages, const int32_t* tile_seq, const int32_t* tile_tok0, const int32_t* tile_ntok, const int32_t* tile_pos0,
                               int n_tiles, int max_tile_tokens, int H, int G, int dk, int dv, float scale, int mask, int mask_size,
                               const float* sink, int n_splits, float* part, int n_tokens, int maps, const float* gate, int ldg,
                               cudaStream_t stream) {
  const size_t smem = ((size_t)TM_KEYS * (dk + 1) + (vcache ? (size_t)TM_KEYS * dv : 0) + (size_t)TM_ROWS * dk + (size_t)TM_ROWS * TM_KEYS) * sizeof(float);
  EL_REFUSE(smem <= 227 * 1024, "masked_attn_tiled: heads of %d / %d need %zu bytes of shared memory", dk, dv, smem);
  auto kern = masked_attn_tiled_kernel<T, TO, NC>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int grp = H / G;
  const dim3 grid(n_tiles, G * maps, ((max_tile_tokens * grp + TM_ROWS - 1) / TM_ROWS) * n_splits);
  const int bit = pdl_bit_for_tokens(n_tokens);
  launch_pdl(bit, kern, grid, dim3(TM_WARPS * 32), smem, stream, q, (TO*)out, (const T*)kcache, (const T*)vcache, page_table, table_stride, n_pages,
             tile_seq, tile_tok0, tile_ntok, tile_pos0, H, G, dk, dv, scale, mask, mask_size, sink, n_splits, part, maps, gate, ldg);
  if (n_splits > 1) {
    if (cudaGetLastError() != cudaSuccess) return 0;   // (the caller reports it)
    launch_pdl(bit, masked_attn_fold_kernel<TO>, dim3(n_tokens, H * maps), dim3(dv >= 256 ? 256 : 128), (size_t)0, stream, (const float*)part, (TO*)out, sink,
               H * maps, dv, n_splits, gate, ldg, maps);
  }
  return 0;
}

extern "C" int edgelm_masked_attn_tiled(const float* q, void* out, int out_dtype, const void* kcache, const void* vcache, int dtype,
                                        const int32_t* page_table, int table_stride, int n_pages, const int32_t* tile_seq,
                                        const int32_t* tile_tok0, const int32_t* tile_ntok, const int32_t* tile_pos0, int n_tiles,
                                        int max_tile_tokens, int H, int G, int dk, int dv, float scale, int mask, int mask_size,
                                        const float* sink, int n_splits, float* part, int n_tokens, int maps, const float* gate, int ldg,
                                        cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  EL_REFUSE(maps >= 1 && G * maps <= 65535 && (maps == 1 || (sink == nullptr && vcache != nullptr)), "masked_attn_tiled: %d maps take no sink and values of their own", maps);
  EL_REFUSE(n_splits >= 1 && n_splits <= 64 && (n_splits == 1 || part != nullptr) && n_tokens > 0, "masked_attn_tiled: %d splits", n_splits);
  if (masked_common_check("masked_attn_tiled", H, G, dk, dv, mask, mask_size, dtype, out_dtype)) return -1;
  EL_REFUSE(n_tiles > 0 && max_tile_tokens > 0 && G <= 65535, "masked_attn_tiled: bad tile counts");
  EL_REFUSE(vcache != nullptr || dv <= dk, "masked_attn_tiled: values of %d inside keys of %d", dv, dk);
  int rc = 0;
#define EL_MT2(T, TO, NC) rc = launch_masked_tiled<T, TO, NC>(q, out, kcache, vcache, page_table, table_stride, n_pages, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, max_tile_tokens, H, G, dk, dv, scale, mask, mask_size, sink, n_splits, part, n_tokens, maps, gate, ldg, stream)
#define EL_MT(NC) do { if (dtype == DT_F32) EL_MT2(float, float, NC); else if (out_dtype == DT_F32) EL_MT2(__nv_bfloat16, float, NC); else EL_MT2(__nv_bfloat16, __nv_bfloat16, NC); } while (0)
  if (dv <= 32) EL_MT(1); else if (dv <= 64) EL_MT(2); else if (dv <= 128) EL_MT(4); else if (dv <= 256) EL_MT(8); else EL_MT(16);
#undef EL_MT
#undef EL_MT2
  if (rc != 0) return rc;
  EL_LAUNCH_CHECK("masked_attn_tiled");
  return 0;
}
