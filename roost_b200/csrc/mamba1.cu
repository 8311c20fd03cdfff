// The Mamba selective scan over a step's rows, with the state of every request in a slot of 32-bit floats:
// [S: inner x state with the state index fastest | the convolution's last taps-1 inputs] (the convolution and its state are the
// kernels of mamba2.cu, which take any channel range).
//
//   scan: per (row, channel c), for the row's tokens in order: dt = softplus(dt_raw[t, c] + dt_bias[c]);
//         S[c, n] <- exp(dt A[c, n]) S[c, n] + dt x[t, c] B[t, n];  y = sum_n S[c, n] C[t, n] + D[c] x[t, c];
//         out[t, c] = y * silu(z[t, c]), rounded once. A is given as it enters the decay (negative), dt_raw is the step
//         projection's 32-bit output, x the convolution's output, [dt | B | C] rows of the projection of x, z the second half
//         of the input projection's rows. S is read from and written to the row's slot. 32-bit throughout.
// A channel's state is shared by L adjacent lanes (L a power of two, each lane keeps 8 state indices in registers); a block
// of 128 threads takes 128 / L channels and stages 8 tokens of B, C, dt and x at a time. The float32 form computes the decay
// exp(dt A) with a reduced-argument polynomial rounded to nearest instead of the special-function unit's exponential: that
// unit's error (up to 2 units in the last place) leans one way for the small arguments of slow decays, and a state multiplied by
// it a thousand times in a row drifts by that lean times a thousand, far above the rounding of everything else. Rows are given by q_indptr (token
// range) and slots; the padding rows of a captured step name a scratch slot. Every sum's order depends on the sizes only.
#include "common.cuh"

namespace roost {

constexpr int kM1Threads = 128;
constexpr int kM1Chunk = 8;
constexpr int kM1PerLane = 8;

// exp(x) for x <= 0 to about one unit in the last place: x = j ln2 + r with ln2 in two parts, a degree-7 polynomial in r.
__device__ __forceinline__ float exp_nearest(float x) {
  if (x < -87.0f) return 0.f;
  const float j = rintf(x * 1.44269504088896341f);
  float r = fmaf(j, -0.693359375f, x);
  r = fmaf(j, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  const float y = fmaf(p * r, r, r) + 1.0f;
  return y * __int_as_float(((int)j + 127) << 23);
}
template <typename T>
__device__ __forceinline__ float decay_exp(float x) { return expf(x); }
template <>
__device__ __forceinline__ float decay_exp<float>(float x) { return exp_nearest(x); }

template <typename T>
__global__ void __launch_bounds__(kM1Threads) mamba1_scan_kernel(const T* __restrict__ xc, const float* __restrict__ dt_raw, const T* __restrict__ dbc,
                                                                int64_t ld_dbc, const T* __restrict__ xz, int64_t ld_xz, T* __restrict__ out,
                                                                const float* __restrict__ dt_bias, const float* __restrict__ a_neg,
                                                                const float* __restrict__ d_skip, float* state, int64_t state_stride,
                                                                const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots, int inner,
                                                                int N, int R, int L) {
  extern __shared__ float sm[];
  const int NP = L * kM1PerLane;                 // state indices, padded
  const int CPB = kM1Threads / L;                // channels a block
  float* sB = sm;                                // [chunk][NP]
  float* sC = sB + kM1Chunk * NP;                // [chunk][NP]
  float* sdt = sC + kM1Chunk * NP;               // [chunk][CPB]
  float* sx = sdt + kM1Chunk * CPB;              // [chunk][CPB]
  float* sy = sx + kM1Chunk * CPB;               // [chunk][CPB]
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int c0 = blockIdx.y * CPB;
  const int cl = threadIdx.x / L, j = threadIdx.x % L;
  const int c = c0 + cl;
  const bool live = c < inner;
  const int n0 = j * kM1PerLane;
  const int start = q_indptr[r], end = q_indptr[r + 1];
  float a[kM1PerLane], S[kM1PerLane];
#pragma unroll
  for (int i = 0; i < kM1PerLane; ++i) a[i] = (live && n0 + i < N) ? a_neg[(size_t)c * N + n0 + i] : 0.f;
  const float skip = live ? d_skip[c] : 0.f;
  float* Sg = state + (size_t)slots[r] * state_stride + (size_t)(live ? c : 0) * N;
  pdl_wait();
  if (end <= start) return;
#pragma unroll
  for (int i = 0; i < kM1PerLane; ++i) S[i] = (live && n0 + i < N) ? Sg[n0 + i] : 0.f;
  for (int t0 = start; t0 < end; t0 += kM1Chunk) {
    const int nt = min(kM1Chunk, end - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * NP; idx += kM1Threads) {
      const int tt = idx / NP, n = idx % NP;
      const T* row = dbc + (size_t)(t0 + tt) * ld_dbc + R;
      sB[idx] = n < N ? to_float(row[n]) : 0.f;
      sC[idx] = n < N ? to_float(row[N + n]) : 0.f;
    }
    for (int idx = threadIdx.x; idx < nt * CPB; idx += kM1Threads) {
      const int tt = idx / CPB, cc = c0 + idx % CPB;
      float dt = 0.f, x = 0.f;
      if (cc < inner) {
        const float zdt = dt_raw[(size_t)(t0 + tt) * inner + cc] + dt_bias[cc];
        dt = zdt > 20.f ? zdt : log1pf(expf(zdt));
        x = to_float(xc[(size_t)(t0 + tt) * inner + cc]);
      }
      sdt[idx] = dt;
      sx[idx] = x;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float dt = sdt[tt * CPB + cl], x = sx[tt * CPB + cl];
      const float dx = dt * x;
      const float* B = sB + tt * NP + n0;
      const float* C = sC + tt * NP + n0;
      float y = 0.f;
#pragma unroll
      for (int i = 0; i < kM1PerLane; ++i) {
        S[i] = fmaf(decay_exp<T>(dt * a[i]), S[i], dx * B[i]);
        y = fmaf(S[i], C[i], y);
      }
      for (int o = L >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (j == 0) sy[tt * CPB + cl] = fmaf(skip, x, y);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * CPB; idx += kM1Threads) {
      const int tt = idx / CPB, cc = c0 + idx % CPB;
      if (cc < inner) {
        const float z = to_float(xz[(size_t)(t0 + tt) * ld_xz + inner + cc]);
        out[(size_t)(t0 + tt) * inner + cc] = from_float<T>(sy[idx] * (z / (1.0f + expf(-z))));
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < kM1PerLane; ++i)
      if (n0 + i < N) Sg[n0 + i] = S[i];
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_mamba1_scan(const void* xc, const float* dt_raw, const void* dbc, int64_t ld_dbc, const void* xz, int64_t ld_xz, void* out,
                                 const float* dt_bias, const float* a_neg, const float* d_skip, float* state, int64_t state_stride,
                                 const int32_t* q_indptr, const int32_t* slots, int rows, int tokens, int inner, int n_state, int dt_rank,
                                 int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && tokens >= 0 && inner > 0 && n_state > 0 && dt_rank > 0, "mamba1_scan: sizes must be positive");
  ROOST_REQUIRE(xc && dt_raw && dbc && xz && out && dt_bias && a_neg && d_skip && state && q_indptr && slots, "mamba1_scan: a pointer is null");
  ROOST_REQUIRE(ld_dbc >= dt_rank + 2 * n_state && ld_xz >= 2 * inner && state_stride >= (int64_t)inner * n_state,
                "mamba1_scan: a row or a slot is too narrow");
  if (n_state > 32 * kM1PerLane) return fail(ROOST_ERR_UNSUPPORTED, "mamba1_scan: a state beyond 256 numbers a channel");
  if (rows == 0 || tokens == 0) return ROOST_OK;
  int L = 1;
  while (L * kM1PerLane < n_state) L *= 2;
  const int cpb = kM1Threads / L;
  const int gy = (inner + cpb - 1) / cpb;
  if (gy > 65535) return fail(ROOST_ERR_UNSUPPORTED, "mamba1_scan: too many channels");
  const size_t smem = ((size_t)2 * kM1Chunk * L * kM1PerLane + (size_t)3 * kM1Chunk * cpb) * sizeof(float);
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(mamba1_scan_kernel<T>, dim3(rows, gy), dim3(kM1Threads), smem, (cudaStream_t)stream, (const T*)xc,
                                               dt_raw, (const T*)dbc, ld_dbc, (const T*)xz, ld_xz, (T*)out, dt_bias, a_neg, d_skip, state,
                                               state_stride, q_indptr, slots, inner, n_state, dt_rank, L));
  return check_launch("mamba1_scan");
}
