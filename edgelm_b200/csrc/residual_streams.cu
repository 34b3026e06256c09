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

template <typename TO>
__global__ void __launch_bounds__(RS_THREADS)
streams_update_kernel(float* __restrict__ xs, const float* __restrict__ y, const float* __restrict__ mix, const float* __restrict__ w_out,
                      const float* __restrict__ w_in, const float* __restrict__ norm_w, float eps, TO* __restrict__ h, int S, int D) {
  pdl_launch_dependents();
  extern __shared__ float rs_u[];        // D floats: the read-out of this token, kept between the two passes
  __shared__ float red[33];
  __shared__ float cm[RS_MAX * RS_MAX], co[RS_MAX], ci[RS_MAX];
  if (threadIdx.x < S * S && y) cm[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < S) {
    co[threadIdx.x] = y ? w_out[threadIdx.x] : 0.f;
    ci[threadIdx.x] = w_in ? w_in[threadIdx.x] : 0.f;
  }
  pdl_wait();
  __syncthreads();
  float* row = xs + (size_t)blockIdx.x * S * D;
  const float* yr = y ? y + (size_t)blockIdx.x * D : nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v[RS_MAX];
#pragma unroll
    for (int s = 0; s < RS_MAX; ++s) v[s] = s < S ? row[(size_t)s * D + d] : 0.f;
    if (yr) {
      const float yv = yr[d];
      float n[RS_MAX];
#pragma unroll
      for (int t = 0; t < RS_MAX; ++t) {
        float a = 0.f;
#pragma unroll
        for (int s = 0; s < RS_MAX; ++s)
          if (s < S && t < S) a = fmaf(cm[s * S + t], v[s], a);
        n[t] = fmaf(co[t < S ? t : 0], yv, a);
      }
#pragma unroll
      for (int t = 0; t < RS_MAX; ++t)
        if (t < S) { v[t] = n[t]; row[(size_t)t * D + d] = n[t]; }
    }
    if (w_in) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < RS_MAX; ++s)
        if (s < S) u = fmaf(ci[s], v[s], u);
      if (norm_w) { rs_u[d] = u; ss = fmaf(u, u, ss); }
      else h[(size_t)blockIdx.x * D + d] = from_f32<TO>(u);
    }
  }
  if (!w_in || !norm_w) return;
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x) h[(size_t)blockIdx.x * D + d] = from_f32<TO>(rs_u[d] * inv * norm_w[d]);
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
  if (h_dtype == DT_BF16) {
    auto kern = streams_update_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(bit, kern, dim3(n_tokens), dim3(RS_THREADS), smem, stream, xs, y, mix, w_out, w_in, norm_w, eps, (__nv_bfloat16*)h, S, D);
  } else if (h_dtype == DT_F32) {
    auto kern = streams_update_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(bit, kern, dim3(n_tokens), dim3(RS_THREADS), smem, stream, xs, y, mix, w_out, w_in, norm_w, eps, (float*)h, S, D);
  } else {
    EL_REFUSE(false, "streams_update: unknown dtype code %d", h_dtype);
  }
  EL_LAUNCH_CHECK("streams_update");
  return 0;
}
