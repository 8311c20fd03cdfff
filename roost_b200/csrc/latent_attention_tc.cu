// Latent attention on the tensor cores for bfloat16 steps of many tokens (prompt portions).
//
// The heads of a token share its keys, so the (token, head) pairs of one request are packed into rows: a block takes 64
// consecutive packed rows, loads their queries [q_latent | q_rot] once, and walks the keys they can see in tiles of 32,
// copied from the pages by cp.async into two buffers. Per tile a warp (16 rows) forms S = Q K^T with mma.sync m16n8k16
// (32-bit accumulators), scales and masks it per row (a row's window is its own token's), keeps the running maximum and
// denominator in 32-bit, and adds P V with V = the first `rank` numbers of the same tile; a weight enters that product as two bfloat16 operands
// (its rounding and the remainder), so that the 32-bit weights are used to 16 bits and not to 8. The sums of a row live in registers: `NT` column tiles of 8 a warp; beyond 256 latent numbers two warps share a
// row group, each with half of the columns and its own copy of S. A block finds its request by walking q_indptr, so the
// kernel needs no list from the host; blocks beyond the step's tiles leave at once.
#include "common.cuh"

namespace roost {

constexpr int kTcRows = 64;
constexpr int kTcKeys = 32;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int NT, int RC>
__global__ void __launch_bounds__(128 * RC) latent_attention_tc_kernel(
    const __nv_bfloat16* __restrict__ q_latent, const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
    const __nv_bfloat16* __restrict__ pool, const int32_t* __restrict__ positions, const int32_t* __restrict__ q_indptr,
    const int32_t* __restrict__ kv_indptr, const int32_t* __restrict__ kv_indices, int tokens, int batch_rows, int heads, int nope, int rope,
    int rank, int page_size, float scale, int window) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int E = rank + rope;
  const int EP = ((E + 15) / 16) * 16;       // k runs in steps of 16: the columns up to EP are zero
  const int LD = EP + 8;                     // row stride in elements: 16 bytes more than a multiple of 32
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [64][LD]
  __nv_bfloat16* Ks = Qs + kTcRows * LD;                                          // [2][32][LD]
  int* rpos = reinterpret_cast<int*>(Ks + 2 * kTcKeys * LD);                      // [64] position of a row's token (-1: no row)
  int* rlo = rpos + kTcRows;                                                      // [64] first key the row sees
  int* item = rlo + kTcRows;                                                      // [2] the block's request and its first packed row
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    int at = 0, found = -1, first = 0;
    for (int b = 0; b < batch_rows; ++b) {
      const int n = (q_indptr[b + 1] - q_indptr[b]) * heads;
      const int t = (n + kTcRows - 1) / kTcRows;
      if ((int)blockIdx.x < at + t) {
        found = b;
        first = ((int)blockIdx.x - at) * kTcRows;
        break;
      }
      at += t;
    }
    item[0] = found;
    item[1] = first;
  }
  __syncthreads();
  const int b = item[0], r0 = item[1];
  if (b < 0) return;
  const int tok0 = q_indptr[b];
  const int n_rows = (q_indptr[b + 1] - tok0) * heads;
  const int32_t* pages = kv_indices + kv_indptr[b];
  pdl_wait();
  // the rows' positions and windows
  for (int r = tid; r < kTcRows; r += blockDim.x) {
    const bool ok = r0 + r < n_rows;
    const int pos = ok ? positions[tok0 + (r0 + r) / heads] : -1;
    rpos[r] = pos;
    rlo[r] = window > 0 ? max(0, pos - window + 1) : 0;
  }
  // the queries: 16-byte pieces of [q_latent | q_rot], zeros for rows beyond the request and for the columns up to LD
  const int pieces = LD / 8;
  for (int idx = tid; idx < kTcRows * pieces; idx += blockDim.x) {
    const int r = idx / pieces, c = (idx % pieces) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r0 + r < n_rows && c < E) {
      const int t = tok0 + (r0 + r) / heads, h = (r0 + r) % heads;
      const __nv_bfloat16* src = c < rank ? q_latent + ((size_t)h * tokens + t) * rank + c
                                          : q + ((size_t)t * heads + h) * (nope + rope) + nope + (c - rank);
      v = *reinterpret_cast<const uint4*>(src);
    }
    *reinterpret_cast<uint4*>(Qs + r * LD + c) = v;
  }
  for (int idx = tid; idx < 2 * kTcKeys * pieces; idx += blockDim.x) {      // the key buffers' columns beyond E stay zero
    const int r = idx / pieces, c = (idx % pieces) * 8;
    if (c >= E) *reinterpret_cast<uint4*>(Ks + r * LD + c) = make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  const int last = min(kTcRows, n_rows - r0) - 1;
  const int kmin = rlo[0], kmax = rpos[last];        // rows are in token order: the first sees furthest back, the last furthest ahead
  if (kmax < 0) return;                               // padding tokens: nobody reads their output

  const int e_pieces = E / 8;
  auto load_tile = [&](int j0, int buf) {
    __nv_bfloat16* dst = Ks + (size_t)buf * kTcKeys * LD;
    for (int idx = tid; idx < kTcKeys * e_pieces; idx += blockDim.x) {
      const int i = idx / e_pieces, c = (idx % e_pieces) * 8;
      const int j = j0 + i;
      if (j >= kmin && j <= kmax) {
        const int page = pages[j / page_size];
        cp16(dst + i * LD + c, pool + ((size_t)page * page_size + (j % page_size)) * E + c);
      } else {
        *reinterpret_cast<uint4*>(dst + i * LD + c) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  const int rg = warp & 3, cs = warp >> 2;            // the warp's 16 rows and its share of the columns
  const int g = lane >> 2, q4 = lane & 3;
  const int row_a = rg * 16 + g, row_b = row_a + 8;
  const int pos_a = rpos[row_a], pos_b = rpos[row_b], lo_a = rlo[row_a], lo_b = rlo[row_b];
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int col0 = cs * NT * 8;                       // the warp's first output column

  const int first_tile = (kmin / kTcKeys) * kTcKeys;
  load_tile(first_tile, 0);
  int buf = 0;
  for (int j0 = first_tile; j0 <= kmax; j0 += kTcKeys, buf ^= 1) {
    if (j0 + kTcKeys <= kmax) {
      load_tile(j0 + kTcKeys, buf ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const __nv_bfloat16* Kt = Ks + (size_t)buf * kTcKeys * LD;
    // S = Q K^T: 16 rows x 32 keys
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    for (int k0 = 0; k0 < EP; k0 += 16) {
      uint32_t a[4], kb[4];
      ldsm_x4(a, Qs + (rg * 16 + (lane & 15)) * LD + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < 2; ++np) {                // 16 keys a load: two tiles of 8
        ldsm_x4(kb, Kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + k0 + ((lane >> 3) & 1) * 8);
        mma_bf16_16816(s[2 * np], a, kb[0], kb[1]);
        mma_bf16_16816(s[2 * np + 1], a, kb[2], kb[3]);
      }
    }
    // scale, mask, running maximum and denominator
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int key = j0 + nt * 8 + q4 * 2 + c;
        s[nt][c] = (key >= lo_a && key <= pos_a) ? s[nt][c] * scale : -INFINITY;
        s[nt][2 + c] = (key >= lo_b && key <= pos_b) ? s[nt][2 + c] * scale : -INFINITY;
        mx_a = fmaxf(mx_a, s[nt][c]);
        mx_b = fmaxf(mx_b, s[nt][2 + c]);
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    const float base_a = mn_a == -INFINITY ? 0.f : mn_a, base_b = mn_b == -INFINITY ? 0.f : mn_b;   // a row that has seen no key yet
    const float corr_a = expf(m_a - base_a), corr_b = expf(m_b - base_b);                          // exp(-inf) = 0 the first time
    m_a = mn_a;
    m_b = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
    uint32_t p[2][4], p_low[2][4];      // a weight as two bfloat16 operands, its rounding and what the rounding left: 16 bits of it
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const float p0 = expf(s[nt][0] - base_a), p1 = expf(s[nt][1] - base_a);
      const float p2 = expf(s[nt][2] - base_b), p3 = expf(s[nt][3] - base_b);
      sum_a += p0 + p1;
      sum_b += p2 + p3;
      const uint32_t hi_a = pack_bf16(p0, p1), hi_b = pack_bf16(p2, p3);
      p[nt >> 1][(nt & 1) * 2] = hi_a;
      p[nt >> 1][(nt & 1) * 2 + 1] = hi_b;
      p_low[nt >> 1][(nt & 1) * 2] = pack_bf16(p0 - __uint_as_float(hi_a << 16), p1 - __uint_as_float(hi_a & 0xffff0000u));
      p_low[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2 - __uint_as_float(hi_b << 16), p3 - __uint_as_float(hi_b & 0xffff0000u));
    }
    l_a = l_a * corr_a + sum_a;
    l_b = l_b * corr_b + sum_b;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      o[i][0] *= corr_a;
      o[i][1] *= corr_a;
      o[i][2] *= corr_b;
      o[i][3] *= corr_b;
    }
    // O += P V, V = the tile's first `rank` columns
#pragma unroll
    for (int kt = 0; kt < 2; ++kt) {
#pragma unroll
      for (int i = 0; i < NT; i += 2) {
        const int d0 = col0 + i * 8;
        if (d0 < rank) {
          uint32_t vb[4];
          ldsm_x4_trans(vb, Kt + (kt * 16 + (lane & 15)) * LD + d0 + (lane >> 4) * 8);
          mma_bf16_16816(o[i], p[kt], vb[0], vb[1]);
          mma_bf16_16816(o[i], p_low[kt], vb[0], vb[1]);
          if (d0 + 8 < rank) {
            mma_bf16_16816(o[i + 1], p[kt], vb[2], vb[3]);
            mma_bf16_16816(o[i + 1], p_low[kt], vb[2], vb[3]);
          }
        }
      }
    }
    __syncthreads();     // the buffer may be filled again
  }
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const float inv_a = l_a > 0.f ? 1.0f / l_a : 0.f, inv_b = l_b > 0.f ? 1.0f / l_b : 0.f;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = r0 + (half ? row_b : row_a);
    if (r >= n_rows) continue;
    const int t = tok0 + r / heads, h = r % heads;
    __nv_bfloat16* dst = out + ((size_t)h * tokens + t) * rank;
    const float inv = half ? inv_b : inv_a;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int d = col0 + i * 8 + q4 * 2;
      if (d < rank) *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16(o[i][half * 2] * inv, o[i][half * 2 + 1] * inv);
    }
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_latent_attention_tc_supported(int nope, int rope, int rank) {
  return nope % 8 == 0 && rope % 8 == 0 && rank % 16 == 0 && rank <= 512 && rank + rope <= 1024;
}

extern "C" int roost_latent_attention_tc(const void* q_latent, const void* q, void* out, const void* pool, const int32_t* positions,
                                         const int32_t* q_indptr, const int32_t* kv_indptr, const int32_t* kv_indices, int tokens,
                                         int batch_rows, int heads, int nope, int rope, int rank, int page_size, float scale, int window,
                                         roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && batch_rows > 0 && heads > 0 && page_size > 0, "latent_attention_tc: sizes must be positive");
  if (!roost_latent_attention_tc_supported(nope, rope, rank)) return fail(ROOST_ERR_UNSUPPORTED, "latent_attention_tc: sizes no tensor-core form serves");
  ROOST_REQUIRE((uintptr_t)q_latent % 16 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)pool % 16 == 0 && (uintptr_t)out % 4 == 0,
                "latent_attention_tc: a pointer is not aligned");
  if (tokens == 0) return ROOST_OK;
  const int E = rank + rope, LD = ((E + 15) / 16) * 16 + 8;
  const size_t smem = ((size_t)kTcRows + 2 * kTcKeys) * LD * 2 + (2 * kTcRows + 4) * sizeof(int);
  if (smem > 220 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "latent_attention_tc: a cache entry too wide for shared memory");
  const long long blocks = ((long long)tokens * heads + kTcRows - 1) / kTcRows + batch_rows;
  if (blocks > 2147483647LL) return fail(ROOST_ERR_UNSUPPORTED, "latent_attention_tc: too many rows");
  using B = __nv_bfloat16;
#define ROOST_LA_TC(NT, RC)                                                                                                           \
  do {                                                                                                                                \
    auto kernel = latent_attention_tc_kernel<NT, RC>;                                                                                 \
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                                            \
    launch_kernel(kernel, dim3((unsigned)blocks), dim3(128 * RC), smem, (cudaStream_t)stream, (const B*)q_latent, (const B*)q, (B*)out, \
                  (const B*)pool, positions, q_indptr, kv_indptr, kv_indices, tokens, batch_rows, heads, nope, rope, rank, page_size, scale, \
                  window);                                                                                                            \
  } while (0)
  if (rank <= 64) ROOST_LA_TC(8, 1);
  else if (rank <= 128) ROOST_LA_TC(16, 1);
  else if (rank <= 256) ROOST_LA_TC(32, 1);
  else ROOST_LA_TC(32, 2);
#undef ROOST_LA_TC
  return check_launch("latent_attention_tc");
}
