// The ends and the norm of a model whose residual stream is kept in 32-bit whatever the activation dtype is: an embedding
// gather that scales (the product formed and stored in 32-bit), a layer norm with weight and bias that first adds a branch
// output to the stream in 32-bit, and the tanh cap of 32-bit logits.
//
// layer norm: y = (x - mean) / sqrt(var + eps) * w + b, var the mean of the squared deviations; mean and var are two
// passes over the row, which a block keeps in shared memory, so that var is a sum of squares of small numbers.
#include "common.cuh"

namespace roost {

template <typename T>
__global__ void embedding_scaled_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids, float* __restrict__ out,
                                        int hidden, int vocab, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  const T* src = table + (size_t)(ok ? id : 0) * hidden;
  float* dst = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? to_float(src[i]) * scale : 0.f;
}

// One block per output row. addend (may be null): s = stream + addend in 32-bit, written back to the stream unless the rows
// are gathered.
template <typename T>
__global__ void layer_norm_kernel(float* stream, const T* __restrict__ addend, const float* __restrict__ w, const float* __restrict__ b,
                                  T* __restrict__ out, const int32_t* __restrict__ rows, int hidden, float eps) {
  extern __shared__ float row[];  // hidden floats, then 32 floats of reduction scratch
  float* scratch = row + hidden;
  pdl_launch_dependents();
  pdl_wait();
  const int i_out = blockIdx.x;
  const size_t r = rows ? (size_t)rows[i_out] : (size_t)i_out;
  float sum = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = stream[r * hidden + i];
    if (addend) {
      v += to_float(addend[r * hidden + i]);
      if (!rows) stream[r * hidden + i] = v;
    }
    row[i] = v;
    sum += v;
  }
  const float mean = block_sum(sum, scratch) / (float)hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float d = row[i] - mean;
    ss += d * d;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)i_out * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<T>((row[i] - mean) * inv * w[i] + b[i]);
}

__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap, float inv_cap) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] * inv_cap);
}

}  // namespace roost

using namespace roost;

extern "C" int roost_embedding_scaled(const void* table, const int32_t* ids, float* out, int tokens, int hidden, int vocab, float scale,
                                      int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embedding_scaled: tokens, hidden and vocab must be positive");
  if (tokens == 0) return ROOST_OK;
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(embedding_scaled_kernel<T>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, (const T*)table, ids,
                                               out, hidden, vocab, scale));
  return check_launch("embedding_scaled");
}

extern "C" int roost_layer_norm(float* stream, const void* addend, const float* w, const float* b, void* out, const int32_t* rows, int n_out,
                                int hidden, float eps, int dtype, roost_stream_t stream_handle) {
  ROOST_REQUIRE(n_out >= 0 && hidden > 0, "layer_norm: rows and hidden must be positive");
  ROOST_REQUIRE(eps > 0.f, "layer_norm: eps must be positive");
  ROOST_REQUIRE(stream && w && b && out, "layer_norm: a pointer is null");
  if (n_out == 0) return ROOST_OK;
  const size_t smem = ((size_t)hidden + 32) * sizeof(float);
  if (smem > 200 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "layer_norm: a row of more than 51168 elements does not fit in shared memory");
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = layer_norm_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, dim3(n_out), dim3(threads), smem, (cudaStream_t)stream_handle, stream, (const T*)addend, w, b, (T*)out, rows, hidden, eps);
  });
  return check_launch("layer_norm");
}

extern "C" int roost_softcap(float* logits, int64_t n, float cap, roost_stream_t stream) {
  ROOST_REQUIRE(n >= 0 && cap > 0.f, "softcap: the count must not be negative and the cap must be positive");
  if (n == 0) return ROOST_OK;
  const int64_t blocks = (n + 255) / 256;
  if (blocks > 2147483647LL) return fail(ROOST_ERR_UNSUPPORTED, "softcap: too many logits for one launch");
  launch_kernel(softcap_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, logits, (size_t)n, cap, 1.0f / cap);
  return check_launch("softcap");
}
