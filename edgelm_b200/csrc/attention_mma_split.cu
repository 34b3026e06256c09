// Causal attention of many new tokens over the paged bfloat16 cache on the tensor cores, for designs whose scores AND softmax
// weights are float32: the float32 operand of each product is written as the sum of three bfloat16 terms (8 + 8 + 8 of its 24
// mantissa bits), each of which the tensor cores multiply exactly with the bfloat16 operand from the cache, sums in float32:
//
//   S = (q1 + q2 + q3) K^T        q float32 queries (after rotation), K bfloat16 cache rows
//   O += (p1 + p2 + p3) V         p float32 softmax weights, V bfloat16 cache rows
//
// so a score or an output differs from the float32 product of the same numbers by float32 rounding only, at three times
// the multiply-adds of a bfloat16 attention instead of the CUDA cores' rate.  Flash style: no score matrix reaches memory.
//
// grid (query tile, query head); a block of 4 warps (times NG groups) owns 64 consecutive new tokens of one sequence for one
// head, 16 rows a warp.  Keys and values are visited page by page (64 positions): all threads of a group copy the page's K
// and V rows of the head's kv head into shared memory with 16-byte cp.async into rows padded by 16 bytes, two stages; K
// fragments by ldmatrix, V fragments by ldmatrix.trans; scale, causal mask, running maximum and sum per row in float32,
// scores in units of log 2.  With NG warp groups a block, group i visits the pages i, i + NG, ... with stages and a named
// barrier of its own; the groups' partial (maximum, sum, output) are merged in shared memory in the order of the groups.
// An optional gate per (token, head) multiplies the head's output by its sigmoid before the rounding.
// Takes key = value head sizes 32, 64, 96, 128, a causal mask, no sink; the page table's rows are the step's sequences.
#include <math_constants.h>

#include "common.cuh"

namespace edgelm {

constexpr int SP_WARPS = 4;
constexpr int SP_ROWS = 16 * SP_WARPS;  // new tokens per block

__device__ __forceinline__ uint32_t sp_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void sp_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void sp_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void sp_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void sp_cp16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// Two float32 values as three packed pairs of bfloat16 terms: x = t1 + t2 + t3 up to float32 rounding (each term the
// rounding of what the terms before left over; the remainders are exact in float32).
__device__ __forceinline__ void sp_split(float x, float y, uint32_t& t1, uint32_t& t2, uint32_t& t3) {
  const __nv_bfloat16 x1 = __float2bfloat16_rn(x), y1 = __float2bfloat16_rn(y);
  const float xr = x - __bfloat162float(x1), yr = y - __bfloat162float(y1);
  const __nv_bfloat16 x2 = __float2bfloat16_rn(xr), y2 = __float2bfloat16_rn(yr);
  const __nv_bfloat16 x3 = __float2bfloat16_rn(xr - __bfloat162float(x2)), y3 = __float2bfloat16_rn(yr - __bfloat162float(y2));
  const __nv_bfloat162 p1 = __halves2bfloat162(x1, y1), p2 = __halves2bfloat162(x2, y2), p3 = __halves2bfloat162(x3, y3);
  t1 = *reinterpret_cast<const uint32_t*>(&p1);
  t2 = *reinterpret_cast<const uint32_t*>(&p2);
  t3 = *reinterpret_cast<const uint32_t*>(&p3);
}

template <int HDT, int NG>  // head size / 16 (even); warp groups that share the pages of a tile
__global__ void __launch_bounds__(SP_WARPS * 32 * NG)
attn_prefill_split_kernel(const float* __restrict__ q, int ldq, __nv_bfloat16* __restrict__ out, int ldo,
                          const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                          const int32_t* __restrict__ page_table, int table_stride, const int32_t* __restrict__ tile_seq,
                          const int32_t* __restrict__ tile_tok0, const int32_t* __restrict__ tile_ntok,
                          const int32_t* __restrict__ tile_pos0, int nh, int nkv, float scale, const float* __restrict__ gate, int ldg) {
  constexpr int HD = HDT * 16;
  constexpr int PITCH = HD + 8;             // elements: 16 bytes of padding per row
  constexpr int CHUNKS = HD / 8;            // 16-byte chunks per row
  extern __shared__ __align__(16) uint8_t sp_raw[];
  constexpr int STAGE = 2 * PAGE * PITCH;
  const int group = threadIdx.x / (SP_WARPS * 32), gtid = threadIdx.x % (SP_WARPS * 32);
  __nv_bfloat16* sm = reinterpret_cast<__nv_bfloat16*>(sp_raw) + (size_t)group * 2 * STAGE;  // this group's [2 stages][K: 64 x PITCH | V: 64 x PITCH]

  const int tile = blockIdx.x, head = blockIdx.y;
  const int g = nh / nkv, kvh = head / g;
  const int lane = threadIdx.x & 31, warp = (threadIdx.x >> 5) % SP_WARPS, gid = lane >> 2, tig = lane & 3;
  const int seq = tile_seq[tile], tok0 = tile_tok0[tile], ntok = tile_ntok[tile], pos0 = tile_pos0[tile];
  const int32_t* pages = page_table + (size_t)seq * table_stride;
  const int nkeys_block = pos0 + ntok;      // keys 0 .. pos0 + ntok - 1
  const int n_pages = (nkeys_block + PAGE - 1) / PAGE;
  const int rowA = warp * 16 + gid, rowB = rowA + 8;      // this lane's two rows (token index inside the tile)
  const int limA = rowA < ntok ? pos0 + rowA : -1;         // last key a row may see; -1: no such row
  const int limB = rowB < ntok ? pos0 + rowB : -1;
  const int warp_limit = min(ntok - 1, warp * 16 + 15) >= warp * 16 ? pos0 + min(ntok - 1, warp * 16 + 15) : -1;
  const int warp_min_limit = warp * 16 < ntok ? pos0 + warp * 16 : -1;   // what the warp's first row sees: pages up to here need no mask
  const float scale2 = scale * 1.4426950408889634f;                     // scores in units of log 2

  auto load_page = [&](int pg, int stage) {
    const int page = pages[pg];
    const __nv_bfloat16* kp = kcache + ((size_t)page * nkv + kvh) * PAGE * HD;
    const __nv_bfloat16* vp = vcache + ((size_t)page * nkv + kvh) * PAGE * HD;
    const int valid = page >= 0 ? min(PAGE, nkeys_block - pg * PAGE) : 0;     // (a page that is not there: zeros, never read)
    __nv_bfloat16* ks = sm + stage * STAGE;
    __nv_bfloat16* vs = ks + PAGE * PITCH;
    for (int i = gtid; i < PAGE * CHUNKS; i += SP_WARPS * 32) {
      const int r = i / CHUNKS, c = i - r * CHUNKS;
      const int bytes = r < valid ? 16 : 0;   // rows past the last key: zero fill, nothing is read
      sp_cp16(sp_smem(ks + r * PITCH + c * 8), bytes ? kp + r * HD + c * 8 : kcache, bytes);
      sp_cp16(sp_smem(vs + r * PITCH + c * 8), bytes ? vp + r * HD + c * 8 : vcache, bytes);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // Q fragments for the whole kernel: three terms of every float32 query value
  uint32_t qa[3][HDT][4];
  {
    const float* qA = q + (size_t)(tok0 + min(rowA, ntok - 1)) * ldq + head * HD;
    const float* qB = q + (size_t)(tok0 + min(rowB, ntok - 1)) * ldq + head * HD;
#pragma unroll
    for (int ks = 0; ks < HDT; ++ks) {
      const int d = ks * 16 + tig * 2;
      const float2 a0 = rowA < ntok ? *reinterpret_cast<const float2*>(qA + d) : make_float2(0.f, 0.f);
      const float2 b0 = rowB < ntok ? *reinterpret_cast<const float2*>(qB + d) : make_float2(0.f, 0.f);
      const float2 a1 = rowA < ntok ? *reinterpret_cast<const float2*>(qA + d + 8) : make_float2(0.f, 0.f);
      const float2 b1 = rowB < ntok ? *reinterpret_cast<const float2*>(qB + d + 8) : make_float2(0.f, 0.f);
      sp_split(a0.x, a0.y, qa[0][ks][0], qa[1][ks][0], qa[2][ks][0]);
      sp_split(b0.x, b0.y, qa[0][ks][1], qa[1][ks][1], qa[2][ks][1]);
      sp_split(a1.x, a1.y, qa[0][ks][2], qa[1][ks][2], qa[2][ks][2]);
      sp_split(b1.x, b1.y, qa[0][ks][3], qa[1][ks][3], qa[2][ks][3]);
    }
  }
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mA = -CUDART_INF_F, mB = -CUDART_INF_F, lA = 0.f, lB = 0.f;

  auto group_sync = [&]() {   // the 128 threads of this group (barrier 0 is __syncthreads)
    if (NG == 1) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(SP_WARPS * 32) : "memory");
  };
  if (group < n_pages) load_page(group, 0);
  for (int pg = group, it = 0; pg < n_pages; pg += NG, ++it) {
    const int stage = it & 1;
    if (pg + NG < n_pages) {
      load_page(pg + NG, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    group_sync();
    if (pg * PAGE <= warp_limit) {   // else: no row of this warp sees this page
      const __nv_bfloat16* ks = sm + stage * STAGE;
      const __nv_bfloat16* vs = ks + PAGE * PITCH;
      // ---- S = Q K^T : 8 tiles of 8 keys, three query terms against every key fragment
      float s[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int ks2 = 0; ks2 < HDT; ks2 += 2) {
          // four 8x8 matrices: (keys nt*8.., d block ks2*16), (.., +8), (.., (ks2+1)*16), (.., +8)
          const int mi = lane >> 3;
          const uint32_t addr = sp_smem(ks + (nt * 8 + (lane & 7)) * PITCH + (ks2 + (mi >> 1)) * 16 + (mi & 1) * 8);
          uint32_t b0, b1, b2, b3;
          sp_ldmatrix_x4(addr, b0, b1, b2, b3);
#pragma unroll
          for (int t = 2; t >= 0; --t) {      // (the small terms first)
            sp_mma(s[nt], qa[t][ks2][0], qa[t][ks2][1], qa[t][ks2][2], qa[t][ks2][3], b0, b1);
            sp_mma(s[nt], qa[t][ks2 + 1][0], qa[t][ks2 + 1][1], qa[t][ks2 + 1][2], qa[t][ks2 + 1][3], b2, b3);
          }
        }
      }
      // ---- scale, causal mask, running max and sum (float32), scores in units of log 2
      const bool masked = pg * PAGE + PAGE - 1 > warp_min_limit;
      float mxA = -CUDART_INF_F, mxB = -CUDART_INF_F;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int key = pg * PAGE + nt * 8 + tig * 2;
        if (masked) {
          s[nt][0] = key <= limA ? s[nt][0] * scale2 : -CUDART_INF_F;
          s[nt][1] = key + 1 <= limA ? s[nt][1] * scale2 : -CUDART_INF_F;
          s[nt][2] = key <= limB ? s[nt][2] * scale2 : -CUDART_INF_F;
          s[nt][3] = key + 1 <= limB ? s[nt][3] * scale2 : -CUDART_INF_F;
        } else {
          s[nt][0] *= scale2;
          s[nt][1] *= scale2;
          s[nt][2] *= scale2;
          s[nt][3] *= scale2;
        }
        mxA = fmaxf(mxA, fmaxf(s[nt][0], s[nt][1]));
        mxB = fmaxf(mxB, fmaxf(s[nt][2], s[nt][3]));
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      const float nmA = fmaxf(mA, mxA), nmB = fmaxf(mB, mxB);
      const float refA = nmA == -CUDART_INF_F ? 0.f : nmA, refB = nmB == -CUDART_INF_F ? 0.f : nmB;  // a row that sees no key yet
      const float corrA = exp2f(mA - refA), corrB = exp2f(mB - refB);  // exp2(-inf) = 0 on the first page
      float sumA = 0.f, sumB = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - refA);
        s[nt][1] = exp2f(s[nt][1] - refA);
        s[nt][2] = exp2f(s[nt][2] - refB);
        s[nt][3] = exp2f(s[nt][3] - refB);
        sumA += s[nt][0] + s[nt][1];
        sumB += s[nt][2] + s[nt][3];
      }
      sumA += __shfl_xor_sync(0xffffffffu, sumA, 1);
      sumA += __shfl_xor_sync(0xffffffffu, sumA, 2);
      sumB += __shfl_xor_sync(0xffffffffu, sumB, 1);
      sumB += __shfl_xor_sync(0xffffffffu, sumB, 2);
      lA = lA * corrA + sumA;
      lB = lB * corrB + sumB;
      mA = nmA;
      mB = nmB;
      if (__any_sync(0xffffffffu, corrA != 1.f || corrB != 1.f)) {   // some row's maximum moved: rescale what is gathered
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
          o[i][0] *= corrA;
          o[i][1] *= corrA;
          o[i][2] *= corrB;
          o[i][3] *= corrB;
        }
      }
      // ---- O += P V : 4 steps of 16 keys, three terms of every weight against every value fragment
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
        uint32_t a[3][4];
        sp_split(s[2 * kt][0], s[2 * kt][1], a[0][0], a[1][0], a[2][0]);
        sp_split(s[2 * kt][2], s[2 * kt][3], a[0][1], a[1][1], a[2][1]);
        sp_split(s[2 * kt + 1][0], s[2 * kt + 1][1], a[0][2], a[1][2], a[2][2]);
        sp_split(s[2 * kt + 1][2], s[2 * kt + 1][3], a[0][3], a[1][3], a[2][3]);
#pragma unroll
        for (int dt = 0; dt < HD / 8; dt += 2) {
          // transposed 8x8 matrices: (keys kt*16.., d block dt), (keys +8, dt), (keys kt*16.., dt+1), (keys +8, dt+1)
          const int mi = lane >> 3;
          const uint32_t addr = sp_smem(vs + (kt * 16 + (mi & 1) * 8 + (lane & 7)) * PITCH + (dt + (mi >> 1)) * 8);
          uint32_t b0, b1, b2, b3;
          sp_ldmatrix_x4_trans(addr, b0, b1, b2, b3);
#pragma unroll
          for (int t = 2; t >= 0; --t) {
            sp_mma(o[dt], a[t][0], a[t][1], a[t][2], a[t][3], b0, b1);
            sp_mma(o[dt + 1], a[t][0], a[t][1], a[t][2], a[t][3], b2, b3);
          }
        }
      }
    }
    group_sync();  // this stage is free for the page after next
  }
  if (NG > 1) {
    // ---- merge the groups: groups 1.. leave (max, sum, output) in shared memory, group 0 folds them in order
    __syncthreads();
    float* mg = reinterpret_cast<float*>(sp_raw);            // [NG - 1][64 rows][HD + 2]
    constexpr int MP = HD + 2;
    if (group > 0) {
      float* a = mg + ((size_t)(group - 1) * SP_ROWS + rowA) * MP;
      float* b = mg + ((size_t)(group - 1) * SP_ROWS + rowB) * MP;
#pragma unroll
      for (int dt = 0; dt < HD / 8; ++dt) {
        a[dt * 8 + tig * 2] = o[dt][0];
        a[dt * 8 + tig * 2 + 1] = o[dt][1];
        b[dt * 8 + tig * 2] = o[dt][2];
        b[dt * 8 + tig * 2 + 1] = o[dt][3];
      }
      if (tig == 0) {
        a[HD] = mA;
        a[HD + 1] = lA;
        b[HD] = mB;
        b[HD + 1] = lB;
      }
    }
    __syncthreads();
    if (group > 0) return;
    for (int gsrc = 1; gsrc < NG; ++gsrc) {
      const float* a = mg + ((size_t)(gsrc - 1) * SP_ROWS + rowA) * MP;
      const float* b = mg + ((size_t)(gsrc - 1) * SP_ROWS + rowB) * MP;
      const float nmA = fmaxf(mA, a[HD]), nmB = fmaxf(mB, b[HD]);
      const float refA = nmA == -CUDART_INF_F ? 0.f : nmA, refB = nmB == -CUDART_INF_F ? 0.f : nmB;
      const float fA0 = exp2f(mA - refA), fA1 = exp2f(a[HD] - refA), fB0 = exp2f(mB - refB), fB1 = exp2f(b[HD] - refB);
      lA = lA * fA0 + a[HD + 1] * fA1;
      lB = lB * fB0 + b[HD + 1] * fB1;
      mA = nmA;
      mB = nmB;
#pragma unroll
      for (int dt = 0; dt < HD / 8; ++dt) {
        o[dt][0] = o[dt][0] * fA0 + a[dt * 8 + tig * 2] * fA1;
        o[dt][1] = o[dt][1] * fA0 + a[dt * 8 + tig * 2 + 1] * fA1;
        o[dt][2] = o[dt][2] * fB0 + b[dt * 8 + tig * 2] * fB1;
        o[dt][3] = o[dt][3] * fB0 + b[dt * 8 + tig * 2 + 1] * fB1;
      }
    }
  }
  float invA = lA > 0.f ? 1.0f / lA : 0.f, invB = lB > 0.f ? 1.0f / lB : 0.f;
  if (gate != nullptr) {      // the head's output gate: sigmoid of its logit
    if (rowA < ntok) invA *= 1.0f / (1.0f + expf(-gate[(size_t)(tok0 + rowA) * ldg + head]));
    if (rowB < ntok) invB *= 1.0f / (1.0f + expf(-gate[(size_t)(tok0 + rowB) * ldg + head]));
  }
#pragma unroll
  for (int dt = 0; dt < HD / 8; ++dt) {
    const int d = head * HD + dt * 8 + tig * 2;
    if (rowA < ntok) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(o[dt][0] * invA, o[dt][1] * invA);
      *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(tok0 + rowA) * ldo + d) = v;
    }
    if (rowB < ntok) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(o[dt][2] * invB, o[dt][3] * invB);
      *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(tok0 + rowB) * ldo + d) = v;
    }
  }
}

template <int HDT, int NG>
static int launch_split_ng(const float* q, int ldq, void* out, int ldo, const void* kc, const void* vc, const int32_t* page_table,
                           int table_stride, const int32_t* tile_seq, const int32_t* tile_tok0, const int32_t* tile_ntok,
                           const int32_t* tile_pos0, int n_tiles, int nh, int nkv, float scale, const float* gate, int ldg,
                           cudaStream_t stream) {
  constexpr int HD = HDT * 16;
  const size_t stages = (size_t)NG * 2 * 2 * PAGE * (HD + 8) * 2, merge = (size_t)(NG - 1) * SP_ROWS * (HD + 2) * 4;
  const size_t smem = stages > merge ? stages : merge;
  auto kern = attn_prefill_split_kernel<HDT, NG>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("attn_prefill_split: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    return -2;
  }
  kern<<<dim3(n_tiles, nh), SP_WARPS * 32 * NG, smem, stream>>>(q, ldq, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
                                                                 page_table, table_stride, tile_seq, tile_tok0, tile_ntok, tile_pos0, nh, nkv, scale,
                                                                 gate, ldg);
  return 0;
}

template <int HDT>
static int launch_split(int groups, const float* q, int ldq, void* out, int ldo, const void* kc, const void* vc, const int32_t* page_table,
                        int table_stride, const int32_t* tile_seq, const int32_t* tile_tok0, const int32_t* tile_ntok,
                        const int32_t* tile_pos0, int n_tiles, int nh, int nkv, float scale, const float* gate, int ldg, cudaStream_t stream) {
#define EL_SP(NG) launch_split_ng<HDT, NG>(q, ldq, out, ldo, kc, vc, page_table, table_stride, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, nh, nkv, scale, gate, ldg, stream)
  if (groups == 2) return EL_SP(2);
  return EL_SP(1);
#undef EL_SP
}

}  // namespace edgelm

using namespace edgelm;

// Tokens per tile that the host must cut sequences into for this kernel.
extern "C" int edgelm_attn_prefill_split_tile_tokens() { return SP_ROWS; }

// 1 if the kernel takes this head size (keys and values alike), else 0.
extern "C" int edgelm_attn_prefill_split_takes(int hd) { return (hd == 32 || hd == 64 || hd == 96 || hd == 128) ? 1 : 0; }

// q [tokens][nh hd] float32 (row pitch ldq), out [tokens][nh hd] bfloat16 (row pitch ldo), the cache bfloat16
// [page][kv head][64][hd]; tiles of at most 64 new tokens of one sequence each; `page_table` rows are the step's sequences
// (tile_seq indexes them).  `gate` (or null): float32 [tokens][>= nh] with row pitch ldg.  `max_keys`: the most keys a tile
// attends over (a hint for how many warp groups share a tile's pages).
extern "C" int edgelm_attn_prefill_split(const float* q, int ldq, void* out, int ldo, const void* kcache, const void* vcache,
                                         const int32_t* page_table, int table_stride, const int32_t* tile_seq, const int32_t* tile_tok0,
                                         const int32_t* tile_ntok, const int32_t* tile_pos0, int n_tiles, int nh, int nkv, int hd,
                                         float scale, const float* gate, int ldg, int max_keys, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  EL_REFUSE(nh > 0 && nkv > 0 && nh % nkv == 0, "attn_prefill_split: %d query heads are not a multiple of %d key/value heads", nh, nkv);
  EL_REFUSE(edgelm_attn_prefill_split_takes(hd), "attn_prefill_split: head size %d (takes 32, 64, 96, 128)", hd);
  EL_REFUSE(ldq % 2 == 0 && ldo % 2 == 0 && (uintptr_t)q % 8 == 0 && (uintptr_t)out % 4 == 0, "attn_prefill_split: rows must be 8- and 4-byte aligned");
  EL_REFUSE((uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0, "attn_prefill_split: the cache must be 16-byte aligned");
  EL_REFUSE(n_tiles > 0 && nh <= 65535, "attn_prefill_split: bad grid");
  const long long blocks = (long long)n_tiles * nh;
  const int groups = ((max_keys + PAGE - 1) / PAGE >= 6 && blocks < 4 * 148 * 2) ? 2 : 1;
  int rc = 0;
  switch (hd / 16) {
    case 2: rc = launch_split<2>(groups, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, nh, nkv, scale, gate, ldg, stream); break;
    case 4: rc = launch_split<4>(groups, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, nh, nkv, scale, gate, ldg, stream); break;
    case 6: rc = launch_split<6>(groups, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, nh, nkv, scale, gate, ldg, stream); break;
    case 8: rc = launch_split<8>(groups, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, nh, nkv, scale, gate, ldg, stream); break;
  }
  if (rc) return rc;
  EL_LAUNCH_CHECK("attn_prefill_split");
  return 0;
}
