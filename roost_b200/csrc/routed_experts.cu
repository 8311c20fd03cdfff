// A feed-forward routed over experts, on the device from the router's logits to the summed outputs.
//
//   router_logits: z[t, e] = x[t, :] . W[e, :], a 32-bit sum whatever the activation dtype is.
//   route:        per token the `top` largest logits choose its experts (ties to the lower index; the sigmoid is monotonic, so the
//                 logits are compared); a pair (token, choice) gets the weight sigmoid(logit). Pairs are sorted by expert:
//                 offsets[e] .. offsets[e+1] are expert e's rows; token_of / weight_of / expert_of give a sorted row's token,
//                 weight and expert; inverse[token * top + k] is where the token's k-th choice went. The sorted rows are also
//                 cut into tiles of kMoeTile rows that meet one expert each: tiles[3n ..] = (expert, first row, one past the last).
//   gather_scale: xs[row, :] = weight_of[row] * x[token_of[row], :], the product formed in 32-bit and rounded once.
//   expert products over the sorted rows: out = silu(xs Wg[e]^T) * (xs Wu[e]^T), or out = act Wd[e]^T. Two forms: tiles of
//                 rows on FFMA (every output sums over k in increasing order in one thread), and, for the few rows of a decode
//                 step, a warp an output that streams the row's expert with 16-byte loads.
//   combine:      out[t, :] = sum_k ys[inverse[t * top + k], :] (+ shared[t, :]), summed in 32-bit in the order of k.
//
// A second form of routing (mode 1): scores are the softmax of the first `experts` logits of a token's row of `columns` logits
// (a row may carry further columns that are not routed); the choice compares score + correction[e], the weight of a pair is
// score * scale; experts from `real` on are identity experts: they get sorted rows like the others but no tiles, the expert
// products skip their rows, and combine_weighted takes the token's own row for them:
//   combine_weighted: out[t, :] = sum_k weight[r_k] * (expert[r_k] < real ? ys[r_k, :] : x[t, :]) (+ sigmoid(gate[t]) * shared[t, :]),
//                 r_k = inverse[t * top + k], summed in 32-bit in the order of k.
// The gated expert product applies the gate function of common.cuh (silu, the tanh form of GELU, the clamped swish).
#include "common.cuh"

#include <mma.h>

namespace roost {

constexpr int kMoeTile = 64;
constexpr int kMoeWideTile = 128;
constexpr int kMoeMaxTop = 32;

// Router logits: a warp a (token, expert), lanes stride over the hidden size with 16-byte loads, 32-bit sums.
template <typename T>
__global__ void __launch_bounds__(256) moe_router_logits_kernel(const T* __restrict__ x, const T* __restrict__ w, float* __restrict__ out,
                                                               int hidden, int experts) {
  constexpr int V = Vec<T>::N;
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.y * 8 + warp;
  pdl_wait();
  if (e >= experts) return;
  const T* xr = x + (size_t)t * hidden;
  const T* wr = w + (size_t)e * hidden;
  float s = 0.f;
  if (hidden % V == 0 && ((uintptr_t)xr % 16 == 0) && ((uintptr_t)wr % 16 == 0)) {
    for (int k = lane * V; k < hidden; k += 32 * V) {
      float av[V], bv[V];
      Vec<T>::load(xr + k, av);
      Vec<T>::load(wr + k, bv);
#pragma unroll
      for (int i = 0; i < V; ++i) s = fmaf(av[i], bv[i], s);
    }
  } else {
    for (int k = lane; k < hidden; k += 32) s = fmaf(to_float(xr[k]), to_float(wr[k]), s);
  }
  s = warp_sum(s);
  if (lane == 0) out[(size_t)t * experts + e] = s;
}

// A warp a token: the token's logits in shared memory, `top` rounds of a warp-wide argmax (ties to the lower index); the
// choice's place among its expert's rows is the expert's running count (the order within an expert is that of arrival:
// every row is computed for itself, so the order changes no value).
__global__ void __launch_bounds__(256) moe_topk_kernel(const float* __restrict__ logits, int tokens, int columns, int experts, int top,
                                                      int mode, const float* __restrict__ correction, float scale,
                                                      int32_t* __restrict__ pair_expert, int32_t* __restrict__ pair_rank,
                                                      float* __restrict__ pair_weight, int32_t* __restrict__ counts) {
  extern __shared__ float zs[];          // [8 warps][experts] what is compared, then [8 warps][experts] the scores (mode 1)
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  pdl_wait();
  if (t >= tokens) return;
  float* z = zs + (size_t)warp * experts;
  float* sc = zs + (size_t)(8 + warp) * experts;
  float zmax = -3.0e38f;
  for (int e = lane; e < experts; e += 32) {
    const float v = logits[(size_t)t * columns + e];
    z[e] = v == v ? fmaxf(v, -3.0e38f) : -3.0e38f;     // a NaN or -inf is the smallest score, not a hole in the order
    zmax = fmaxf(zmax, z[e]);
  }
  if (mode == 1) {       // softmax scores over all routed columns; the choice sees score + correction
    zmax = warp_max(zmax);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) {
      const float ev = expf(z[e] - zmax);
      sc[e] = ev;
      sum += ev;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < experts; e += 32) {
      const float score = sc[e] * inv;
      sc[e] = score * scale;
      z[e] = score + (correction != nullptr ? correction[e] : 0.f);
    }
  }
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    float bz = -INFINITY;
    int best = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = z[e];
      if (v > bz) {
        bz = v;
        best = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float oz = __shfl_xor_sync(0xffffffffu, bz, o);
      const int ob = __shfl_xor_sync(0xffffffffu, best, o);
      if (oz > bz || (oz == bz && ob < best)) {
        bz = oz;
        best = ob;
      }
    }
    if (lane == 0) {
      z[best] = -INFINITY;               // taken
      pair_expert[(size_t)t * top + k] = best;
      pair_rank[(size_t)t * top + k] = atomicAdd(&counts[best], 1);
      if (mode == 1) pair_weight[(size_t)t * top + k] = sc[best];
    }
    __syncwarp();
  }
}

// One block: the experts' counts become their row ranges and the list of tiles, every pair goes to its sorted row, and the
// counts are left at zero for the next call.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const float* __restrict__ logits, int tokens, int columns, int experts, int real, int top,
                                                       int mode, const float* __restrict__ pair_weight,
                                                       int32_t* __restrict__ token_of, float* __restrict__ weight_of,
                                                       int32_t* __restrict__ expert_of, int32_t* __restrict__ inverse,
                                                       int32_t* __restrict__ offsets, int32_t* __restrict__ tiles, int max_tiles,
                                                       int32_t* __restrict__ wide_tiles, int max_wide_tiles,
                                                       const int32_t* __restrict__ pair_expert, const int32_t* __restrict__ pair_rank,
                                                       int32_t* __restrict__ counts) {
  extern __shared__ int32_t offs[];      // [experts + 1]
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int at = 0, n = 0;
    for (int e = 0; e < experts; ++e) {
      const int c = counts[e];
      offs[e] = at;
      offsets[e] = at;
      for (int r = at; r < at + c && e < real; r += kMoeTile) {
        tiles[3 * n] = e;
        tiles[3 * n + 1] = r;
        tiles[3 * n + 2] = min(r + kMoeTile, at + c);
        ++n;
      }
      at += c;
    }
    offs[experts] = at;
    offsets[experts] = at;
    for (; n < max_tiles; ++n) tiles[3 * n] = -1;
  }
  if (threadIdx.x == 32 && wide_tiles != nullptr) {      // the same rows in tiles of kMoeWideTile, for the tcgen05 product
    int at = 0, n = 0;
    for (int e = 0; e < experts; ++e) {
      const int c = counts[e];
      for (int r = at; r < at + c && e < real; r += kMoeWideTile) {
        wide_tiles[3 * n] = e;
        wide_tiles[3 * n + 1] = r;
        wide_tiles[3 * n + 2] = min(r + kMoeWideTile, at + c);
        ++n;
      }
      at += c;
    }
    for (; n < max_wide_tiles; ++n) wide_tiles[3 * n] = -1;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  for (int i = threadIdx.x; i < tokens * top; i += blockDim.x) {
    const int e = pair_expert[i];
    const int dest = offs[e] + pair_rank[i];
    const float z = logits[(size_t)(i / top) * columns + e];
    token_of[dest] = i / top;
    weight_of[dest] = mode == 1 ? pair_weight[i] : 1.0f / (1.0f + expf(-z));
    expert_of[dest] = e;
    inverse[i] = dest;
  }
}

template <typename T>
__global__ void moe_gather_scale_kernel(const T* __restrict__ x, T* __restrict__ xs, const int32_t* __restrict__ token_of,
                                        const float* __restrict__ weight_of, int hidden, int scaled) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const T* src = x + (size_t)token_of[row] * hidden;
  const float w = weight_of[row];
  if (!scaled) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs[(size_t)row * hidden + i] = src[i];
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs[(size_t)row * hidden + i] = from_float<T>(w * to_float(src[i]));
}

// Gate and up weights come either as two tensors [experts, N, K] (block 0) or as one [experts, 2 N, K] in which an expert's rows
// are interleaved in blocks of `block` gate rows followed by their `block` up rows (the layout of the tcgen05 product's
// activation epilogue): output n's gate row is then (n / block) * 2 * block + n % block and its up row `block` rows on.
template <typename T>
__device__ __forceinline__ const T* moe_expert_base(const T* w, int e, int N, int K, int block) {
  return w + (size_t)e * (block ? 2 : 1) * N * K;
}
__device__ __forceinline__ size_t moe_weight_row(int n, int block) {
  return block ? (size_t)(n / block) * 2 * block + n % block : (size_t)n;
}

// Tiles of 64 sorted rows x 64 outputs of the tile's expert; k in steps of 16. GATED: two weights share the rows and the output
// is silu(a Wg^T) * (a Wu^T).
template <typename T, bool GATED>
__global__ void __launch_bounds__(256) moe_tile_gemm_kernel(const T* __restrict__ a, const T* __restrict__ w1, const T* __restrict__ w2,
                                                           T* __restrict__ out, const int32_t* __restrict__ tiles, int N, int K, int block, int act,
                                                           float limit) {
  constexpr int BM = kMoeTile, BN = 64, BK = 16;
  __shared__ float as[BK][BM + 1];
  __shared__ float ws1[BK][BN + 1];
  __shared__ float ws2[GATED ? BK : 1][BN + 1];
  pdl_launch_dependents();
  pdl_wait();
  const int e = tiles[3 * blockIdx.y];
  if (e < 0) return;
  const int m0 = tiles[3 * blockIdx.y + 1], m_end = tiles[3 * blockIdx.y + 2];
  const int n0 = blockIdx.x * BN;
  const T* wa = moe_expert_base(w1, e, N, K, block);
  const T* wb = GATED ? (block ? wa + (size_t)block * K : w2 + (size_t)e * N * K) : nullptr;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  float acc1[4][4], acc2[GATED ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc1[i][j] = 0.f;
      if (GATED) acc2[i][j] = 0.f;
    }
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int row = idx >> 4, col = idx & 15;
      const int k = k0 + col, m = m0 + row, n = n0 + row;
      as[col][row] = (m < m_end && k < K) ? to_float(a[(size_t)m * K + k]) : 0.f;
      const size_t wr = moe_weight_row(n, block);
      ws1[col][row] = (n < N && k < K) ? to_float(wa[wr * K + k]) : 0.f;
      if (GATED) ws2[col][row] = (n < N && k < K) ? to_float(wb[wr * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[4], bv[4], cv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = as[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        bv[j] = ws1[kk][tx * 4 + j];
        if (GATED) cv[j] = ws2[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc1[i][j] = fmaf(av[i], bv[j], acc1[i][j]);
          if (GATED) acc2[i][j] = fmaf(av[i], cv[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= m_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc1[i][j];
      if (GATED) v = gate_fn(v, acc2[i][j], act, limit);     // on the 32-bit sums
      out[(size_t)m * N + n] = from_float<T>(v);
    }
  }
}

// The same rows on the tensor cores for bfloat16 (mma.sync through the wmma fragments, 32-bit accumulators): a block takes a
// tile of 64 sorted rows and 128 outputs, four warps with 64 x 32 each (a fragment of the rows serves two or four products);
// k in steps of 32 through three stages of shared memory filled by cp.async. Needs k a multiple of 8 (16-byte pieces of whole
// rows). A warp's accumulators leave through a patch of shared memory of its own, where the gated form applies
// silu(gate) * up to the two 32-bit sums.
__device__ __forceinline__ void moe_cp16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}

constexpr int kMoeTcBN = 128, kMoeTcBK = 32, kMoeTcLD = kMoeTcBK + 8, kMoeTcStages = 3;
constexpr int moe_tc_stage_elems(bool gated) { return (kMoeTile + (gated ? 2 : 1) * kMoeTcBN) * kMoeTcLD; }

template <bool GATED>
__global__ void __launch_bounds__(128) moe_tile_gemm_tc_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w1,
                                                              const __nv_bfloat16* __restrict__ w2, __nv_bfloat16* __restrict__ out,
                                                              const int32_t* __restrict__ tiles, int N, int K, int block, int act, float limit) {
  using namespace nvcuda;
  constexpr int BM = kMoeTile, BN = kMoeTcBN, BK = kMoeTcBK, LD = kMoeTcLD, STAGE = moe_tc_stage_elems(GATED);
  extern __shared__ __align__(128) unsigned char raw[];
  __nv_bfloat16* stages = reinterpret_cast<__nv_bfloat16*>(raw);
  pdl_launch_dependents();
  pdl_wait();
  const int e = tiles[3 * blockIdx.y];
  if (e < 0) return;
  const int m0 = tiles[3 * blockIdx.y + 1], m_end = tiles[3 * blockIdx.y + 2];
  const int n0 = blockIdx.x * BN;
  const __nv_bfloat16* wa = moe_expert_base(w1, e, N, K, block);
  const __nv_bfloat16* wb = GATED ? (block ? wa + (size_t)block * K : w2 + (size_t)e * N * K) : nullptr;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto fill = [&](int k0, int st) {
    __nv_bfloat16* As = stages + (size_t)st * STAGE;
    __nv_bfloat16* W1s = As + BM * LD;
    __nv_bfloat16* W2s = W1s + BN * LD;
    if (k0 < K) {
      for (int idx = tid; idx < (BM + (GATED ? 2 : 1) * BN) * 4; idx += 128) {       // 16-byte pieces: four a row
        const int row = idx >> 2, k = k0 + (idx & 3) * 8;
        __nv_bfloat16* dst = As + row * LD + (idx & 3) * 8;        // the three tiles lie back to back with one row stride
        const __nv_bfloat16* src = nullptr;
        if (k < K) {
          if (row < BM) src = m0 + row < m_end ? a + (size_t)(m0 + row) * K + k : nullptr;
          else if (row < BM + BN) src = n0 + row - BM < N ? wa + moe_weight_row(n0 + row - BM, block) * K + k : nullptr;
          else src = n0 + row - BM - BN < N ? wb + moe_weight_row(n0 + row - BM - BN, block) * K + k : nullptr;
        }
        if (src) moe_cp16(dst, src);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc1[4][2], acc2[GATED ? 4 : 1][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      wmma::fill_fragment(acc1[i][j], 0.f);
      if (GATED) wmma::fill_fragment(acc2[i][j], 0.f);
    }
  fill(0, 0);
  fill(BK, 1);
  int st = 0;
  for (int k0 = 0; k0 < K; k0 += BK) {
    fill(k0 + 2 * BK, (st + 2) % kMoeTcStages);        // an empty group beyond k keeps the count of groups in step
    asm volatile("cp.async.wait_group 2;\n" ::);
    __syncthreads();
    const __nv_bfloat16* As = stages + (size_t)st * STAGE;
    const __nv_bfloat16* W1s = As + BM * LD;
    const __nv_bfloat16* W2s = W1s + BN * LD;
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa[4];
      wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb[2], fc[GATED ? 2 : 1];
#pragma unroll
      for (int i = 0; i < 4; ++i) wmma::load_matrix_sync(fa[i], As + (i * 16) * LD + kk, LD);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        wmma::load_matrix_sync(fb[j], W1s + (warp * 32 + j * 16) * LD + kk, LD);
        if (GATED) wmma::load_matrix_sync(fc[j], W2s + (warp * 32 + j * 16) * LD + kk, LD);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          wmma::mma_sync(acc1[i][j], fa[i], fb[j], acc1[i][j]);
          if (GATED) wmma::mma_sync(acc2[i][j], fa[i], fc[j], acc2[i][j]);
        }
    }
    __syncthreads();      // the stage may be filled again
    st = (st + 1) % kMoeTcStages;
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  __syncthreads();
  // a warp's patch: two 16 x 16 blocks of floats with rows of 20
  float* patch = reinterpret_cast<float*>(raw) + warp * 2 * 16 * 20;
  const int pr = lane >> 1, pc = (lane & 1) * 8;        // a lane's row of the block and its eight columns
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      wmma::store_matrix_sync(patch, acc1[i][j], 20, wmma::mem_row_major);
      if (GATED) wmma::store_matrix_sync(patch + 16 * 20, acc2[i][j], 20, wmma::mem_row_major);
      __syncwarp();
      const int m = m0 + i * 16 + pr, n = n0 + warp * 32 + j * 16 + pc;
      if (m < m_end) {
        float v[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          v[c] = patch[pr * 20 + pc + c];
          if (GATED) v[c] = gate_fn(v[c], patch[16 * 20 + pr * 20 + pc + c], act, limit);     // on the 32-bit sums
        }
        __nv_bfloat16* dst = out + (size_t)m * N + n;
        if (n + 8 <= N && N % 8 == 0) {
          Vec<__nv_bfloat16>::store(dst, v);
        } else {
          for (int c = 0; c < 8 && n + c < N; ++c) dst[c] = __float2bfloat16_rn(v[c]);
        }
      }
      __syncwarp();
    }
}

// Few rows: a block per sorted row and 8 outputs, a warp an output; lanes stride over k.
template <typename T, bool GATED>
__global__ void __launch_bounds__(256) moe_row_gemm_kernel(const T* __restrict__ a, const T* __restrict__ w1, const T* __restrict__ w2,
                                                          T* __restrict__ out, const int32_t* __restrict__ expert_of, int N, int K, int block, int act,
                                                          float limit, int real) {
  constexpr int V = Vec<T>::N;
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.y * 8 + warp;
  pdl_wait();
  if (n >= N) return;
  const int e = expert_of[row];
  if (e >= real) return;              // an identity expert has no weights; nobody reads its row of the output
  const T* ar = a + (size_t)row * K;
  const T* wr1 = moe_expert_base(w1, e, N, K, block) + moe_weight_row(n, block) * K;
  const T* wr2 = GATED ? (block ? wr1 + (size_t)block * K : w2 + ((size_t)e * N + n) * K) : nullptr;
  float s1 = 0.f, s2 = 0.f;
  if (K % V == 0 && ((uintptr_t)ar % 16 == 0) && ((uintptr_t)wr1 % 16 == 0) && (!GATED || (uintptr_t)wr2 % 16 == 0)) {
    for (int k = lane * V; k < K; k += 32 * V) {
      float av[V], bv[V];
      Vec<T>::load(ar + k, av);
      Vec<T>::load(wr1 + k, bv);
#pragma unroll
      for (int i = 0; i < V; ++i) s1 = fmaf(av[i], bv[i], s1);
      if (GATED) {
        Vec<T>::load(wr2 + k, bv);
#pragma unroll
        for (int i = 0; i < V; ++i) s2 = fmaf(av[i], bv[i], s2);
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float av = to_float(ar[k]);
      s1 = fmaf(av, to_float(wr1[k]), s1);
      if (GATED) s2 = fmaf(av, to_float(wr2[k]), s2);
    }
  }
  s1 = warp_sum(s1);
  if (GATED) s2 = warp_sum(s2);
  if (lane == 0) {
    float v = s1;
    if (GATED) v = gate_fn(s1, s2, act, limit);     // on the 32-bit sums
    out[(size_t)row * N + n] = from_float<T>(v);
  }
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ ys, const int32_t* __restrict__ inverse, const T* __restrict__ shared,
                                   T* __restrict__ out, int hidden, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc += to_float(ys[(size_t)inverse[(size_t)t * top + k] * hidden + i]);
    if (shared) acc += to_float(shared[(size_t)t * hidden + i]);
    out[(size_t)t * hidden + i] = from_float<T>(acc);
  }
}

template <typename T>
__global__ void moe_combine_weighted_kernel(const T* __restrict__ ys, const int32_t* __restrict__ inverse, const float* __restrict__ weight_of,
                                            const int32_t* __restrict__ expert_of, const T* __restrict__ x, const T* __restrict__ shared,
                                            const float* __restrict__ gate, int gate_stride, T* __restrict__ out, int hidden, int top, int real) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  __shared__ int32_t rk[kMoeMaxTop];
  __shared__ float wk[kMoeMaxTop];
  __shared__ int idk[kMoeMaxTop];
  if (threadIdx.x < top) {
    const int r = inverse[(size_t)t * top + threadIdx.x];
    rk[threadIdx.x] = r;
    wk[threadIdx.x] = weight_of[r];
    idk[threadIdx.x] = expert_of[r] >= real;
  }
  __syncthreads();
  const float g = (shared != nullptr && gate != nullptr) ? 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride])) : 1.0f;
  constexpr int V = Vec<T>::N;
  if (hidden % V == 0 && (uintptr_t)ys % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 && (shared == nullptr || (uintptr_t)shared % 16 == 0)) {
    for (int i = threadIdx.x * V; i < hidden; i += blockDim.x * V) {      // whole 16-byte vectors: the same sums in the same order
      float acc[V], xv[V], v[V];
      Vec<T>::load(x + (size_t)t * hidden + i, xv);
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] = 0.f;
      for (int k = 0; k < top; ++k) {
        if (!idk[k]) Vec<T>::load(ys + (size_t)rk[k] * hidden + i, v);
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = fmaf(wk[k], idk[k] ? xv[e] : v[e], acc[e]);
      }
      if (shared) {
        Vec<T>::load(shared + (size_t)t * hidden + i, v);
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = fmaf(g, v[e], acc[e]);
      }
      Vec<T>::store(out + (size_t)t * hidden + i, acc);
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float acc = 0.f;
    const float xv = to_float(x[(size_t)t * hidden + i]);
    for (int k = 0; k < top; ++k) acc = fmaf(wk[k], idk[k] ? xv : to_float(ys[(size_t)rk[k] * hidden + i]), acc);
    if (shared) acc = fmaf(g, to_float(shared[(size_t)t * hidden + i]), acc);
    out[(size_t)t * hidden + i] = from_float<T>(acc);
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_moe_tile_rows(void) { return kMoeTile; }

extern "C" int roost_moe_router_logits(const void* x, const void* w, float* out, int tokens, int hidden, int experts, int dtype,
                                       roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && hidden > 0 && experts > 0, "moe_router_logits: sizes must be positive");
  if (tokens == 0) return ROOST_OK;
  dim3 grid(tokens, (experts + 7) / 8);
  if (grid.y > 65535) return fail(ROOST_ERR_UNSUPPORTED, "moe_router_logits: too many experts");
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(moe_router_logits_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, (const T*)x, (const T*)w, out,
                                               hidden, experts));
  return check_launch("moe_router_logits");
}

// counts: int32[experts], zero on entry and left at zero (a caller keeps one buffer for all its calls on a stream).
extern "C" int roost_moe_wide_tile_rows(void) { return kMoeWideTile; }

// mode 0: sigmoid scores, compared by logit; mode 1: softmax scores over the `experts` routed columns of a row of `columns`,
// compared with `correction` (may be null) added, weights times `scale`. Experts from `real` on have no tiles. scratch: 3 * tokens *
// top 32-bit words.
extern "C" int roost_moe_route(const float* logits, int tokens, int columns, int experts, int real, int top, int mode, const float* correction,
                               float scale, int32_t* token_of, float* weight_of, int32_t* expert_of, int32_t* inverse, int32_t* offsets,
                               int32_t* tiles, int max_tiles, int32_t* wide_tiles, int max_wide_tiles, int32_t* scratch, int32_t* counts,
                               roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && top <= experts && columns >= experts && real >= 0 && real <= experts,
                "moe_route: sizes do not fit");
  ROOST_REQUIRE(mode == 0 || mode == 1, "moe_route: the mode is 0 (sigmoid) or 1 (softmax)");
  if (top > kMoeMaxTop || experts > 4096) return fail(ROOST_ERR_UNSUPPORTED, "moe_route: more than 32 choices a token or 4096 experts");
  ROOST_REQUIRE((int64_t)max_tiles >= ((int64_t)tokens * top + kMoeTile - 1) / kMoeTile + experts, "moe_route: the tile list is too short");
  ROOST_REQUIRE(counts != nullptr && scratch != nullptr, "moe_route: a pointer is null");
  ROOST_REQUIRE(wide_tiles == nullptr || (int64_t)max_wide_tiles >= ((int64_t)tokens * top + kMoeWideTile - 1) / kMoeWideTile + experts,
                "moe_route: the list of wide tiles is too short");
  if (tokens == 0) return ROOST_OK;
  int32_t* pair_expert = scratch;
  int32_t* pair_rank = scratch + (size_t)tokens * top;
  float* pair_weight = reinterpret_cast<float*>(scratch + (size_t)2 * tokens * top);
  launch_kernel(moe_topk_kernel, dim3((tokens + 7) / 8), dim3(256), (size_t)16 * experts * sizeof(float), (cudaStream_t)stream, logits, tokens,
                columns, experts, top, mode, correction, scale, pair_expert, pair_rank, pair_weight, counts);
  launch_kernel(moe_sort_kernel, dim3(1), dim3(1024), ((size_t)experts + 1) * sizeof(int32_t), (cudaStream_t)stream, logits, tokens, columns, experts,
                real, top, mode, (const float*)pair_weight, token_of, weight_of, expert_of, inverse, offsets, tiles, max_tiles, wide_tiles, max_wide_tiles, (const int32_t*)pair_expert,
                (const int32_t*)pair_rank, counts);
  return check_launch("moe_route");
}

extern "C" int roost_moe_gather_scale(const void* x, void* xs, const int32_t* token_of, const float* weight_of, int rows, int hidden, int scaled,
                                      int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && hidden > 0, "moe_gather_scale: sizes must be positive");
  if (rows == 0) return ROOST_OK;
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(moe_gather_scale_kernel<T>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (const T*)x, (T*)xs,
                                               token_of, weight_of, hidden, scaled));
  return check_launch("moe_gather_scale");
}

// form 0: tiles of rows (tiles: the route's list of max_tiles entries); form 1: a warp an output (expert_of: a sorted row's expert).
// block > 0: the gated product's weights are one tensor, w1 = [experts, 2 n, k] with gate and up rows interleaved in blocks of
// `block` (w2 is then only a flag: any non-null value).
extern "C" int roost_moe_expert_gemm(const void* a, const void* w1, const void* w2, void* out, const int32_t* tiles, int max_tiles,
                                     const int32_t* expert_of, int rows, int n, int k, int form, int block, int act, float limit, int real,
                                     int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && n > 0 && k > 0 && (form == 0 || form == 1), "moe_expert_gemm: sizes do not fit");
  ROOST_REQUIRE(act >= ROOST_ACT_SILU && act <= ROOST_ACT_CLAMPED_SWISH && (act != ROOST_ACT_CLAMPED_SWISH || limit > 0.f || w2 == nullptr),
                "moe_expert_gemm: unknown gate function, or a clamped swish without its limit");
  ROOST_REQUIRE(block >= 0 && (block == 0 || (w2 != nullptr && n % block == 0)), "moe_expert_gemm: an interleave block must divide n and belongs to the gated form");
  if (block) w2 = w1;
  if (rows == 0) return ROOST_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (form == 0) {
    dim3 grid((n + 63) / 64, max_tiles);
    if (max_tiles > 65535) return fail(ROOST_ERR_UNSUPPORTED, "moe_expert_gemm: more than 65535 tiles of rows");
    if (dtype == ROOST_BF16 && k % 8 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)w1 % 16 == 0 && (uintptr_t)w2 % 16 == 0 &&
        (uintptr_t)out % 16 == 0) {
      using B = __nv_bfloat16;
      dim3 tc_grid((n + kMoeTcBN - 1) / kMoeTcBN, max_tiles);
      const size_t smem = (size_t)kMoeTcStages * moe_tc_stage_elems(w2 != nullptr) * sizeof(B);
      if (w2) {
        cudaFuncSetAttribute(moe_tile_gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_kernel(moe_tile_gemm_tc_kernel<true>, tc_grid, dim3(128), smem, s, (const B*)a, (const B*)w1, (const B*)w2, (B*)out, tiles, n, k, block, act, limit);
      } else {
        cudaFuncSetAttribute(moe_tile_gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_kernel(moe_tile_gemm_tc_kernel<false>, tc_grid, dim3(128), smem, s, (const B*)a, (const B*)w1, (const B*)w2, (B*)out, tiles, n, k, block, act, limit);
      }
      return check_launch("moe_expert_gemm");
    }
    ROOST_DISPATCH_DTYPE(dtype, T, {
      if (w2) launch_kernel(moe_tile_gemm_kernel<T, true>, grid, dim3(256), 0, s, (const T*)a, (const T*)w1, (const T*)w2, (T*)out, tiles, n, k, block, act, limit);
      else launch_kernel(moe_tile_gemm_kernel<T, false>, grid, dim3(256), 0, s, (const T*)a, (const T*)w1, (const T*)w2, (T*)out, tiles, n, k, block, act, limit);
    });
  } else {
    dim3 grid(rows, (n + 7) / 8);
    if (grid.y > 65535) return fail(ROOST_ERR_UNSUPPORTED, "moe_expert_gemm: too many outputs");
    ROOST_DISPATCH_DTYPE(dtype, T, {
      if (w2) launch_kernel(moe_row_gemm_kernel<T, true>, grid, dim3(256), 0, s, (const T*)a, (const T*)w1, (const T*)w2, (T*)out, expert_of, n, k, block, act, limit, real);
      else launch_kernel(moe_row_gemm_kernel<T, false>, grid, dim3(256), 0, s, (const T*)a, (const T*)w1, (const T*)w2, (T*)out, expert_of, n, k, block, act, limit, real);
    });
  }
  return check_launch("moe_expert_gemm");
}

extern "C" int roost_moe_combine(const void* ys, const int32_t* inverse, const void* shared, void* out, int tokens, int hidden, int top, int dtype,
                                 roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && hidden > 0 && top > 0, "moe_combine: sizes must be positive");
  if (tokens == 0) return ROOST_OK;
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(moe_combine_kernel<T>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, (const T*)ys, inverse,
                                               (const T*)shared, (T*)out, hidden, top));
  return check_launch("moe_combine");
}

extern "C" int roost_moe_combine_weighted(const void* ys, const int32_t* inverse, const float* weight_of, const int32_t* expert_of, const void* x,
                                          const void* shared, const float* gate, int gate_stride, void* out, int tokens, int hidden, int top,
                                          int real, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && hidden > 0 && top > 0 && top <= kMoeMaxTop, "moe_combine_weighted: sizes do not fit");
  ROOST_REQUIRE(ys && inverse && weight_of && expert_of && x && out, "moe_combine_weighted: a pointer is null");
  if (tokens == 0) return ROOST_OK;
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(moe_combine_weighted_kernel<T>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, (const T*)ys, inverse,
                                               weight_of, expert_of, (const T*)x, (const T*)shared, gate, gate_stride, (T*)out, hidden, top, real));
  return check_launch("moe_combine_weighted");
}
