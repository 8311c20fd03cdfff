// Several 32-bit residual streams a token (hyper-connections), and the gate functions of gated feed-forwards.
//
//   stream_step: streams [tokens, S, width] float32. For an output row i (token t = rows ? rows[i] : i), per channel c:
//                  x_s = init_from ? init_from[t, c] (every stream a copy; stored) : streams[t, s, c]
//                  with y:   x'_r = sum_s mix[s, r] x_s + write[r] y[t, c]   (every stream from the old ones; stored unless rows)
//                  u = read ? sum_s read[s] x'_s : sum_s x'_s
//                out[i, :] = u / sqrt(mean(u^2) + eps) * norm_w      (norm_w float32, any offset folded in), rounded once.
//                One pass over a token's streams does the write-back of the sublayer before and the read of the one ahead.
//   gated_act_mul: out[t, i] = fn(gate[t, i], up[t, i]) over rows [gate | up] or blocks of `block` gate then `block` up values;
//                fn is the gate function of common.cuh (silu, the tanh form of GELU, the clamped swish with its limit).
#include "common.cuh"

namespace roost {

constexpr int kMaxStreams = 8;

template <typename T, int S>
__global__ void __launch_bounds__(512) stream_step_kernel(float* streams, const T* __restrict__ y, const T* __restrict__ init_from,
                                                         const float* __restrict__ mix, const float* __restrict__ write,
                                                         const float* __restrict__ read, const float* __restrict__ norm_w,
                                                         const int32_t* __restrict__ rows, T* __restrict__ out, int width, float eps) {
  extern __shared__ float sm[];          // [width] the read u, then 32 floats of scratch
  float* su = sm;
  float* scratch = sm + width;
  pdl_launch_dependents();
  float mx[S][S], wr[S], rd[S];
#pragma unroll
  for (int s = 0; s < S; ++s) {
    rd[s] = read != nullptr ? read[s] : 1.0f;
    wr[s] = write != nullptr ? write[s] : 0.f;
#pragma unroll
    for (int r = 0; r < S; ++r) mx[s][r] = mix != nullptr ? mix[s * S + r] : 0.f;
  }
  pdl_wait();
  const int i_out = blockIdx.x;
  const size_t t = rows != nullptr ? (size_t)rows[i_out] : (size_t)i_out;
  float* xt = streams + t * S * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float xs[S];
    if (init_from != nullptr) {
      const float v = to_float(init_from[t * width + c]);
#pragma unroll
      for (int s = 0; s < S; ++s) {
        xs[s] = v;
        xt[(size_t)s * width + c] = v;
      }
    } else {
#pragma unroll
      for (int s = 0; s < S; ++s) xs[s] = xt[(size_t)s * width + c];
    }
    if (y != nullptr) {
      const float yv = to_float(y[t * width + c]);
      float nx[S];
#pragma unroll
      for (int r = 0; r < S; ++r) {
        float a = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) a = fmaf(mx[s][r], xs[s], a);
        nx[r] = fmaf(wr[r], yv, a);
      }
#pragma unroll
      for (int r = 0; r < S; ++r) {
        xs[r] = nx[r];
        if (rows == nullptr) xt[(size_t)r * width + c] = nx[r];
      }
    }
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < S; ++s) u = fmaf(rd[s], xs[s], u);
    su[c] = u;
    ss = fmaf(u, u, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  T* o = out + (size_t)i_out * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = from_float<T>(su[c] * inv * norm_w[c]);
}

template <typename T>
__global__ void gated_act_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, int block, int act, float limit) {
  const size_t t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (i >= inter) return;
  const size_t g_at = block ? (size_t)(i / block) * 2 * block + i % block : (size_t)i;
  const size_t u_at = block ? g_at + block : (size_t)inter + i;
  const float g = to_float(x[t * 2 * inter + g_at]);
  const float u = to_float(x[t * 2 * inter + u_at]);
  out[t * inter + i] = from_float<T>(gate_fn(g, u, act, limit));
}

// The same over rows [gate | up] whose halves are whole 16-byte vectors: a thread takes one vector of each.
template <typename T>
__global__ void gated_act_mul_vec_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, int act, float limit) {
  constexpr int V = Vec<T>::N;
  const size_t t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  pdl_launch_dependents();
  pdl_wait();
  if (i >= inter) return;
  float g[V], u[V];
  Vec<T>::load(x + t * 2 * inter + i, g);
  Vec<T>::load(x + t * 2 * inter + inter + i, u);
#pragma unroll
  for (int e = 0; e < V; ++e) g[e] = gate_fn(g[e], u[e], act, limit);
  Vec<T>::store(out + t * inter + i, g);
}

template <typename T, int S>
static cudaError_t launch_stream_step(float* streams, const void* y, const void* init_from, const float* mix, const float* write,
                                      const float* read, const float* norm_w, const int32_t* rows, void* out, int n_out, int width, float eps,
                                      cudaStream_t stream) {
  const size_t smem = ((size_t)width + 32) * sizeof(float);
  auto kernel = stream_step_kernel<T, S>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  // few rows (decode steps): twice the threads a token, half the trips to memory one after the other
  const int threads = n_out <= 64 && width > 256 ? 512 : 256;
  return launch_kernel(kernel, dim3(n_out), dim3(threads), smem, stream, streams, (const T*)y, (const T*)init_from, mix, write, read, norm_w, rows,
                       (T*)out, width, eps);
}

}  // namespace roost

using namespace roost;

extern "C" int roost_stream_step(float* streams, const void* y, const void* init_from, const float* mix, const float* write, const float* read,
                                 const float* norm_w, const int32_t* rows, void* out, int n_out, int n_streams, int width, float eps, int dtype,
                                 roost_stream_t stream) {
  ROOST_REQUIRE(n_out >= 0 && width > 0 && eps > 0.f, "stream_step: rows, width and eps must be positive");
  ROOST_REQUIRE(streams && norm_w && out, "stream_step: a pointer is null");
  ROOST_REQUIRE((y == nullptr) == (mix == nullptr) && (y == nullptr) == (write == nullptr), "stream_step: a write-back needs y, mix and write together");
  ROOST_REQUIRE(!(y != nullptr && init_from != nullptr), "stream_step: fresh streams have no write-back pending");
  ROOST_REQUIRE(!(rows != nullptr && init_from != nullptr), "stream_step: fresh streams are made for every token");
  if (n_streams < 1 || n_streams > kMaxStreams) return fail(ROOST_ERR_UNSUPPORTED, "stream_step: 1 to 8 streams");
  if ((size_t)width * 4 > 200 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "stream_step: a width beyond 51200");
  if (n_out == 0) return ROOST_OK;
#define ROOST_STREAMS_CASE(SN)                                                                                                              \
  case SN:                                                                                                                                  \
    ROOST_DISPATCH_DTYPE(dtype, T, launch_stream_step<T, SN>(streams, y, init_from, mix, write, read, norm_w, rows, out, n_out, width, eps, \
                                                            (cudaStream_t)stream));                                                        \
    break;
  switch (n_streams) {
    ROOST_STREAMS_CASE(1) ROOST_STREAMS_CASE(2) ROOST_STREAMS_CASE(3) ROOST_STREAMS_CASE(4) ROOST_STREAMS_CASE(5) ROOST_STREAMS_CASE(6)
    ROOST_STREAMS_CASE(7) ROOST_STREAMS_CASE(8)
  }
#undef ROOST_STREAMS_CASE
  return check_launch("stream_step");
}

extern "C" int roost_gated_act_mul(const void* x, void* out, int tokens, int inter, int block, int act, float limit, int dtype,
                                   roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && inter > 0, "gated_act_mul: tokens and inter must be positive");
  ROOST_REQUIRE(block == 0 || inter % block == 0, "gated_act_mul: the interleave block must divide inter");
  ROOST_REQUIRE(act >= ROOST_ACT_SILU && act <= ROOST_ACT_CLAMPED_SWISH, "gated_act_mul: unknown gate function");
  ROOST_REQUIRE(act != ROOST_ACT_CLAMPED_SWISH || limit > 0.f, "gated_act_mul: the clamped swish needs a positive limit");
  if (tokens == 0) return ROOST_OK;
  if ((inter + 255) / 256 > 65535) return fail(ROOST_ERR_UNSUPPORTED, "gated_act_mul: inter beyond 16776960");
  const int vec = dtype == ROOST_F32 ? 4 : 8;
  if (block == 0 && inter % vec == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0) {
    dim3 vgrid(tokens, (inter / vec + 127) / 128);
    ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(gated_act_mul_vec_kernel<T>, vgrid, dim3(128), 0, (cudaStream_t)stream, (const T*)x, (T*)out, inter,
                                                 act, limit));
    return check_launch("gated_act_mul");
  }
  dim3 grid(tokens, (inter + 255) / 256);
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(gated_act_mul_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, (const T*)x, (T*)out, inter, block,
                                               act, limit));
  return check_launch("gated_act_mul");
}
