// A residual stream kept as S copies ("hyper-connections"): xs [tokens][S][D] float32.
//
// A sublayer reads u = sum_s w_in[s] xs[s] and its output y [tokens][D] is written back into every stream at once, from
// the old values: xs'[t] = sum_s mix[s][t] xs[s] + w_out[t] y.  One kernel does a write, a read, or a write followed by
// the next sublayer's read, so that the streams make one trip through memory between two sublayers:
//   y given       the write (mix [S][S] indexed [from][to], w_out [S])
//   w_in given    the read, from the new values: with norm_w the RMS norm of u times norm_w goes to `h` in the compute
//                 type (the next matrix product's input); without it u itself goes to `h` as float32 (the plain sum of
//                 the streams when w_in is all ones)
// `streams_fill` starts every stream as a copy of x [tokens][D].  Everything is float32; sums run in a fixed order.
#include "common.cuh"

namespace edgelm {

constexpr int RS_MAX = 8;          // streams at most
constexpr int RS_THREADS = 256;

__global__ void streams_fill_kernel(const float* __restrict__ x, float* __restrict__ xs, int S, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const float* row = x + (size_t)blockIdx.x * D;
  float* dst = xs + (size_t)blockIdx.x * S * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float v = row[d];
    for (int s = 0; s < S; ++s) dst[(size_t)s * D + d] = v;
  }
}

// V floats at once (V 4 when rows are 16-byte aligned, else 1); SM: the unrolled loops' bound on the streams (S <= SM)
template <int V> struct RsVec { float e[V]; };
template <int V> __device__ __forceinline__ RsVec<V> rs_load(const float* p) {
  RsVec<V> r;
  if constexpr (V == 4) { const float4 q = *reinterpret_cast<const float4*>(p); r.e[0] = q.x; r.e[1] = q.y; r.e[2] = q.z; r.e[3] = q.w; }
  else r.e[0] = *p;
  return r;
}
template <int V> __device__ __forceinline__ void rs_store(float* p, const RsVec<V>& r) {
  if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(r.e[0], r.e[1], r.e[2], r.e[3]);
  else *p = r.e[0];
}
template <int V> __device__ __forceinline__ void rs_store(__nv_bfloat16* p, const RsVec<V>& r) {
  if constexpr (V == 4) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(r.e[0], r.e[1]), hi = __floats2bfloat162_rn(r.e[2], r.e[3]);
    uint2 q;
    q.x = *reinterpret_cast<const unsigned*>(&lo);
    q.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = q;
  } else *p = __float2bfloat16(r.e[0]);
}

template <typename TO, int V, int SM>
__global__ void __launch_bounds__(RS_THREADS)
streams_update_kernel(float* __restrict__ xs, const float* __restrict__ y, const float* __restrict__ mix, const float* __restrict__ w_out,
                      const float* __restrict__ w_in, const float* __restrict__ norm_w, float eps, TO* __restrict__ h, int S, int D) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) float rs_u[];        // D floats: the read-out of this token, kept between the two passes
  __shared__ float red[33];
  __shared__ float cm[SM * SM], co[SM], ci[SM];
  // (weights past S are zero: the unrolled sums run to SM)
  if (threadIdx.x < SM * SM) {
    const int f = threadIdx.x / SM, t = threadIdx.x % SM;
    cm[threadIdx.x] = (y && f < S && t < S) ? mix[f * S + t] : 0.f;
  }
  if (threadIdx.x < SM) {
    co[threadIdx.x] = (y && threadIdx.x < S) ? w_out[threadIdx.x] : 0.f;
    ci[threadIdx.x] = (w_in && threadIdx.x < S) ? w_in[threadIdx.x] : 0.f;
  }
  pdl_wait();
  __syncthreads();
  float* row = xs + (size_t)blockIdx.x * S * D;
  const float* yr = y ? y + (size_t)blockIdx.x * D : nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
    RsVec<V> v[SM];
#pragma unroll
    for (int s = 0; s < SM; ++s) {
      if (s < S) v[s] = rs_load<V>(row + (size_t)s * D + d);
      else
#pragma unroll
        for (int e = 0; e < V; ++e) v[s].e[e] = 0.f;
    }
    if (yr) {
      const RsVec<V> yv = rs_load<V>(yr + d);
      RsVec<V> n[SM];
#pragma unroll
      for (int t = 0; t < SM; ++t)
#pragma unroll
        for (int e = 0; e < V; ++e) {
          float a = 0.f;
#pragma unroll
          for (int s = 0; s < SM; ++s) a = fmaf(cm[s * SM + t], v[s].e[e], a);
          n[t].e[e] = fmaf(co[t], yv.e[e], a);
        }
#pragma unroll
      for (int t = 0; t < SM; ++t)
        if (t < S) { v[t] = n[t]; rs_store<V>(row + (size_t)t * D + d, n[t]); }
    }
    if (w_in) {
      RsVec<V> u;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        float a = 0.f;
#pragma unroll
        for (int s = 0; s < SM; ++s) a = fmaf(ci[s], v[s].e[e], a);
        u.e[e] = a;
        ss = fmaf(a, a, ss);
      }
      if (norm_w) rs_store<V>(rs_u + d, u);
      else rs_store<V>(h + (size_t)blockIdx.x * D + d, u);
    }
  }
  if (!w_in || !norm_w) return;
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)D + eps);
  for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
    RsVec<V> u = rs_load<V>(rs_u + d);
    const RsVec<V> w = rs_load<V>(norm_w + d);
#pragma unroll
    for (int e = 0; e < V; ++e) u.e[e] = u.e[e] * inv * w.e[e];
    rs_store<V>(h + (size_t)blockIdx.x * D + d, u);
  }
}

}  // namespace edgelm

using namespace edgelm;

extern "C" int edgelm_streams_fill(const float* x, float* xs, int n_tokens, int S, int D, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && S >= 1 && S <= RS_MAX && D > 0, "streams_fill: %d streams of %d values are not taken (up to %d streams)", S, D, RS_MAX);
  launch_pdl(pdl_bit_for_tokens(n_tokens), streams_fill_kernel, dim3(n_tokens), dim3(D >= 1024 ? 256 : 128), (size_t)0, stream, x, xs, S, D);
  EL_LAUNCH_CHECK("streams_fill");
  return 0;
}

// y (with mix, w_out) null: no write.  w_in null: no read.  norm_w null: `h` receives the read-out itself, float32.
extern "C" int edgelm_streams_update(float* xs, const float* y, const float* mix, const float* w_out, const float* w_in, const float* norm_w,
                                     float eps, void* h, int h_dtype, int n_tokens, int S, int D, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && S >= 1 && S <= RS_MAX && D > 0, "streams_update: %d streams of %d values are not taken (up to %d streams)", S, D, RS_MAX);
  EL_REFUSE((y == nullptr) == (mix == nullptr) && (y == nullptr) == (w_out == nullptr), "streams_update: a write needs y, mix and w_out");
  EL_REFUSE(y != nullptr || w_in != nullptr, "streams_update: neither a write nor a read");
  EL_REFUSE(w_in == nullptr || h != nullptr, "streams_update: a read needs its output");
  EL_REFUSE(norm_w != nullptr || w_in == nullptr || h_dtype == DT_F32, "streams_update: the plain read-out is float32");
  const size_t smem = (w_in && norm_w) ? (size_t)D * sizeof(float) : 0;
  EL_REFUSE(smem <= 200 * 1024, "streams_update: rows of %d values are not taken", D);
  const int bit = pdl_bit_for_tokens(n_tokens);
  EL_REFUSE(h == nullptr || h_dtype == DT_BF16 || h_dtype == DT_F32, "streams_update: unknown dtype code %d", h_dtype);
  // four values at once where every row starts on 16 bytes (8 for a bfloat16 read-out)
  const bool vec = D % 4 == 0 && (uintptr_t)xs % 16 == 0 && (y == nullptr || (uintptr_t)y % 16 == 0) && (norm_w == nullptr || (uintptr_t)norm_w % 16 == 0) &&
                   (h == nullptr || (uintptr_t)h % 16 == 0);
  const int sm = S <= 2 ? 2 : S <= 4 ? 4 : 8;
#define EL_RS(TO, V, SM) do { auto kern = streams_update_kernel<TO, V, SM>; \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    launch_pdl(bit, kern, dim3(n_tokens), dim3(RS_THREADS), smem, stream, xs, y, mix, w_out, w_in, norm_w, eps, (TO*)h, S, D); } while (0)
#define EL_RS_V(TO, V) do { if (sm == 2) EL_RS(TO, V, 2); else if (sm == 4) EL_RS(TO, V, 4); else EL_RS(TO, V, 8); } while (0)
  if (h_dtype == DT_BF16) { if (vec) EL_RS_V(__nv_bfloat16, 4); else EL_RS_V(__nv_bfloat16, 1); }
  else { if (vec) EL_RS_V(float, 4); else EL_RS_V(float, 1); }
#undef EL_RS_V
#undef EL_RS
  EL_LAUNCH_CHECK("streams_update");
  return 0;
}
