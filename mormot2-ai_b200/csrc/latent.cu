// Latent attention on the CUDA cores, for float32 and bfloat16 storage with float32
// arithmetic: the kernels around a cache that keeps ONE row per token, the normed key/value
// latent c (kv_rank values) followed by the rotated key part that all heads share (rot_dim
// values), instead of keys and values per head.
//
// Heads never see keys or values of their own. With k_h = [W_uk,h c ; r] and v_h = W_uv,h c,
//   q_h · k_h = (W_uk,hᵀ q_h,plain) · c + q_h,rot · r        and
//   sum_j p_j v_h,j = W_uv,h (sum_j p_j c_j),
// so the query is carried into the latent space once per token (heads_gemm with W_uk,hᵀ),
// every head attends over the same rows [c ; r] (latent_attention), and the weighted latent
// is carried out again (heads_gemm with W_uv,h). Scores, softmax, norms and angles are float32.
//
//   latent_prep       RMSNorm of the query latent and of the key/value latent, rotation of
//                     the shared key part, the cache row's write
//   heads_gemm        C[t, h, :] = B[h] · A[t, h, :] for every head, a batch of small products;
//                     optionally the rotation of a tail of A that is copied behind C's
//                     columns, or a sigmoid gate on C
//   latent_attention  causal softmax attention of every head over the rows of the cache
#include "common.cuh"
#include "mma_tile.cuh"

MB_DEFINE_LAST_ERROR

// Rotates value i of a part whose first rot_dims values turn (rotate-half pairing: i with
// i + rot_dims/2); the rest pass. buf holds the part in float32. The angle is the float32
// product of the position and the frequency; cosine and sine are multiplied by `amplitude`.
__device__ __forceinline__ float rotated(const float* buf, int i, int rot_dims,
                                         const float* __restrict__ inv_freq, int pos,
                                         float amplitude) {
  if (i >= rot_dims) return buf[i];
  const int half = rot_dims >> 1;
  const int f = i < half ? i : i - half;
  const float angle = inv_freq[f] * (float)pos;
  float s, c;
  sincosf(angle, &s, &c);
  s *= amplitude;
  c *= amplitude;
  return i < half ? buf[i] * c - buf[i + half] * s : buf[i] * c + buf[i - half] * s;
}

// ------------------------------------------------------------------ latent_prep
// f [T, ld]: per token the query latent (q_rank values at column q_col), the key/value latent
// (kv_rank values at column kv_col) and behind it the shared key part (rot_dim values).
// cq_out [T, q_rank] = w_q · rmsnorm(query latent); the cache row of the token's slot and
// position = [w_kv · rmsnorm(key/value latent) ; rotate(shared key part)].
// With parts > 0 the rows are read from `partial` [parts][T, ld] (float32, the split sums of
// the product that made them, added up here in split order) instead of f, and gate_n further
// columns from gate_col on are added up too and written to gate_out [T, gate_n].
template <typename T, typename TW>
__global__ void __launch_bounds__(512)
latent_prep_kernel(const T* __restrict__ f, int ld, int q_col, int kv_col, int q_rank, int kv_rank,
                   int rot_dim, const TW* __restrict__ w_q, const TW* __restrict__ w_kv, float eps,
                   const float* __restrict__ inv_freq, int rot_dims, float amplitude,
                   const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                   const int* __restrict__ page_table, int max_pages, int ring_pages,
                   T* __restrict__ pool, T* __restrict__ cq_out, int write_cache,
                   const float* __restrict__ partial, int parts, size_t part_stride,
                   T* __restrict__ gate_out, int gate_col, int gate_n) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ float buf[];  // q_rank + kv_rank + rot_dim
  __shared__ float red[33];
  const int t = blockIdx.x;
  const T* row = f + (size_t)t * ld;
  const float* prow = partial + (size_t)t * ld;
  auto value = [&](int col) -> float {
    if (parts == 0) return to_f32<T>(row[col]);
    return sum_parts(prow + col, parts, part_stride);
  };
  float* bq = buf;
  float* bc = buf + q_rank;
  float* br = bc + kv_rank;
  float sq = 0.f, sc = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float v = value(q_col + i);
    bq[i] = v;
    sq = fmaf(v, v, sq);
  }
  for (int i = threadIdx.x; i < kv_rank + rot_dim; i += blockDim.x) {
    const float v = value(kv_col + i);
    bc[i] = v;
    if (i < kv_rank) sc = fmaf(v, v, sc);
  }
  if (parts > 0 && gate_out)
    for (int i = threadIdx.x; i < gate_n; i += blockDim.x)
      gate_out[(size_t)t * gate_n + i] = from_f32<T>(value(gate_col + i));
  sq = block_sum(sq, red);
  sc = block_sum(sc, red);
  if (q_rank > 0) {
    const float inv = 1.0f / sqrtf(sq / (float)q_rank + eps);
    T* out = cq_out + (size_t)t * q_rank;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      out[i] = from_f32<T>(to_f32<TW>(w_q[i]) * (bq[i] * inv));
  }
  if (!write_cache) return;
  const int pos = tok_pos[t];
  T* dst = pool + kv_row(page_table, max_pages, ring_pages, tok_slot[t], pos, 1, 0) *
                      (size_t)(kv_rank + rot_dim);
  const float inv = 1.0f / sqrtf(sc / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x)
    dst[i] = from_f32<T>(to_f32<TW>(w_kv[i]) * (bc[i] * inv));
  for (int i = threadIdx.x; i < rot_dim; i += blockDim.x)
    dst[kv_rank + i] = from_f32<T>(rotated(br, i, rot_dims, inv_freq, pos, amplitude));
}

MB_EXPORT int mb_latent_prep(const void* f, int dtype, int ld, int q_col, int kv_col, int q_rank,
                             int kv_rank, int rot_dim, const void* w_q, const void* w_kv,
                             int w_dtype, float eps, const float* inv_freq, int rot_dims,
                             float amplitude, const int* tok_slot, const int* tok_pos,
                             const int* page_table, int max_pages, int ring_pages, void* pool,
                             void* cq_out, int T, int write_cache, const float* partial,
                             int parts, long long part_stride, void* gate_out, int gate_col,
                             int gate_n, void* stream) {
  if (T <= 0) return 0;
  if ((parts > 0) != (partial != nullptr) || (parts == 0 && f == nullptr))
    MB_FAIL("mb_latent_prep: rows or their split sums");
  if (rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1))
    MB_FAIL("mb_latent_prep: %d rotating values of %d", rot_dims, rot_dim);
  if (rot_dims > 0 && inv_freq == nullptr) MB_FAIL("mb_latent_prep: no frequencies");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = (size_t)(q_rank + kv_rank + rot_dim) * sizeof(float);
  if (smem > 48 * 1024) MB_FAIL("mb_latent_prep: latents of %d values", q_rank + kv_rank + rot_dim);
#define GO(T_, TW_)                                                                          \
  mb_launch(latent_prep_kernel<T_, TW_>, dim3(T), dim3(parts > 0 ? 512 : 128), smem, s,      \
            (const T_*)f, ld, q_col,                                                          \
            kv_col, q_rank, kv_rank, rot_dim, (const TW_*)w_q, (const TW_*)w_kv, eps, inv_freq, \
            rot_dims, amplitude, tok_slot, tok_pos, page_table, max_pages, ring_pages,       \
            (T_*)pool, (T_*)cq_out, write_cache, partial, parts, (size_t)part_stride,        \
            (T_*)gate_out, gate_col, gate_n)
  if (dtype == MB_F32) {
    if (w_dtype == MB_F32) GO(float, float); else GO(float, __nv_bfloat16);
  } else {
    if (w_dtype == MB_F32) GO(__nv_bfloat16, float); else GO(__nv_bfloat16, __nv_bfloat16);
  }
#undef GO
  MB_CHECK_LAUNCH("mb_latent_prep");
}

// ------------------------------------------------------------------ heads_gemm
// C[t, h·ldc_h + n] = sum_k A[t·lda + h·lda_h + k] · B[(h·N + n)·K + k] for n < N, every head h
// and token t: one small product per head, the heads a grid dimension. BM tokens x 64 outputs
// a block of 256 threads, float32 multiply-adds.
//   gate != null: C is multiplied by sigmoid(gate[t·ldg + h·N + n]).
//   tail > 0: the `tail` values of A behind the K that are multiplied (A[.., K .. K+tail))
//   are rotated by the token's position (rotated()) and stored behind C's N columns.
#define HG_BN 64
#define HG_BK 16
template <typename T, typename TB, int BM>
__global__ void __launch_bounds__(256)
heads_gemm_kernel(const T* __restrict__ A, int lda, int lda_h, const TB* __restrict__ B,
                  T* __restrict__ C, int ldc, int ldc_h, int M, int N, int K,
                  const T* __restrict__ gate, int ldg, int tail, int rot_dims,
                  const float* __restrict__ inv_freq, float amplitude,
                  const int* __restrict__ tok_pos) {
  mb_grid_wait();
  mb_grid_launch_next();
  constexpr int TM = BM / 16;
  __shared__ float As[HG_BK][BM + 4];
  __shared__ float Bs[HG_BK][HG_BN + 4];
  const int tid = threadIdx.x;
  const int h = blockIdx.z;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * HG_BN;
  const T* Ah = A + (size_t)h * lda_h;
  const TB* Bh = B + (size_t)h * N * K;
  const int tr = (tid / 16) * TM, tc = (tid % 16) * 4;
  float acc[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HG_BK) {
    for (int e = tid; e < BM * HG_BK; e += 256) {
      const int r = e / HG_BK, c = e % HG_BK;
      const int gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_f32<T>(Ah[(size_t)gm * lda + gk]) : 0.f;
    }
    for (int e = tid; e < HG_BN * HG_BK; e += 256) {
      const int r = e / HG_BK, c = e % HG_BK;
      const int gn = n0 + r, gk = k0 + c;
      Bs[c][r] = (gn < N && gk < K) ? to_f32<TB>(Bh[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HG_BK; ++k) {
      float a[TM], b[4];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][tr + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tc + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + tr + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tc + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (gate) {
        const float g = to_f32<T>(gate[(size_t)gm * ldg + (size_t)h * N + gn]);
        v *= 1.0f / (1.0f + expf(-g));
      }
      C[(size_t)gm * ldc + (size_t)h * ldc_h + gn] = from_f32<T>(v);
    }
  }
  if (tail > 0 && blockIdx.x == 0) {
    // As is free again: the tails of up to HG_BK * (BM + 4) / tail rows at a time
    float* tb = &As[0][0];
    const int rows_at_once = max(1, (HG_BK * (BM + 4)) / tail);
    for (int r0 = 0; r0 < BM; r0 += rows_at_once) {
      const int rows = min(rows_at_once, BM - r0);
      __syncthreads();
      for (int e = tid; e < rows * tail; e += 256) {
        const int r = e / tail, i = e % tail;
        const int gm = m0 + r0 + r;
        tb[e] = gm < M ? to_f32<T>(Ah[(size_t)gm * lda + K + i]) : 0.f;
      }
      __syncthreads();
      for (int e = tid; e < rows * tail; e += 256) {
        const int r = e / tail, i = e % tail;
        const int gm = m0 + r0 + r;
        if (gm < M)
          C[(size_t)gm * ldc + (size_t)h * ldc_h + N + i] =
              from_f32<T>(rotated(tb + r * tail, i, rot_dims, inv_freq, tok_pos[gm], amplitude));
      }
    }
  }
}

// The same product on the tensor cores for bfloat16 operands (mma_tile.cuh): a block computes
// 128 tokens x 128 outputs of one head. The gate and the rotated tail as above (the tail is
// read from global memory, value and partner).
__global__ void __launch_bounds__(MT_THREADS)
heads_gemm_mma_kernel(const __nv_bfloat16* __restrict__ A, int lda, int lda_h,
                      const __nv_bfloat16* __restrict__ B, __nv_bfloat16* __restrict__ C, int ldc,
                      int ldc_h, int M, int N, int K, const __nv_bfloat16* __restrict__ gate,
                      int ldg, int tail, int rot_dims, const float* __restrict__ inv_freq,
                      float amplitude, const int* __restrict__ tok_pos) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ __align__(16) MtShared<1> sh;
  constexpr int MT_BN = 128;
  const int h = blockIdx.z, m0 = blockIdx.y * MT_BM, n0 = blockIdx.x * MT_BN;
  const __nv_bfloat16* Ah = A + (size_t)h * lda_h;
  if (threadIdx.x < MT_BM) {
    const int gm = m0 + threadIdx.x;
    sh.a_rows[threadIdx.x] = gm < M ? Ah + (size_t)gm * lda : nullptr;
  }
  __syncthreads();
  const __nv_bfloat16* b[1] = {B + ((size_t)h * N + n0) * K};
  float acc[1][2][8][4];
  mt_mainloop<1>(sh, b, min(MT_BN, N - n0), K, acc);
  mt_for_each<1>([&](int r, int c, int mi, int ni, int e) {
    const int gm = m0 + r, gn = n0 + c;
    if (gm >= M || gn >= N) return;
    float v = acc[0][mi][ni][e];
    if (gate) {
      const float gv = __bfloat162float(gate[(size_t)gm * ldg + (size_t)h * N + gn]);
      v *= 1.0f / (1.0f + expf(-gv));
    }
    C[(size_t)gm * ldc + (size_t)h * ldc_h + gn] = __float2bfloat16_rn(v);
  });
  if (tail > 0 && blockIdx.x == 0) {
    const int half = rot_dims >> 1;
    for (int e = threadIdx.x; e < MT_BM * tail; e += blockDim.x) {
      const int r = e / tail, i = e % tail;
      const int gm = m0 + r;
      if (gm >= M) continue;
      const __nv_bfloat16* src = Ah + (size_t)gm * lda + K;
      float v = __bfloat162float(src[i]);
      if (i < rot_dims) {
        const int f = i < half ? i : i - half;
        float sn, cs;
        sincosf(inv_freq[f] * (float)tok_pos[gm], &sn, &cs);
        sn *= amplitude;
        cs *= amplitude;
        const float other = __bfloat162float(src[i < half ? i + half : i - half]);
        v = i < half ? v * cs - other * sn : v * cs + other * sn;
      }
      C[(size_t)gm * ldc + (size_t)h * ldc_h + N + i] = __float2bfloat16_rn(v);
    }
  }
}

// The same product for a decode step of at most 16 tokens (bfloat16, K a multiple of 32): the
// head's WEIGHT rows are the 16 rows of the m16n8k16 product and the tokens its columns (two
// groups of eight). A warp owns 16 output features over all of K and reads its weight rows
// straight from global memory into the product's registers, 16 bytes a thread and row, several
// steps of K in flight; the tokens' rows of the head wait in shared memory. Within a step of 32
// values of K a thread holds values 8t .. 8t+7 of both operands: the products pair them up in
// another order than the instruction's own, which is the same sum.
#define HR_WARPS 4
__global__ void __launch_bounds__(HR_WARPS * 32)
heads_rows_mma_kernel(const __nv_bfloat16* __restrict__ A, int lda, int lda_h,
                      const __nv_bfloat16* __restrict__ B, __nv_bfloat16* __restrict__ C, int ldc,
                      int ldc_h, int M, int N, int K, const __nv_bfloat16* __restrict__ gate,
                      int ldg, int tail, int rot_dims, const float* __restrict__ inv_freq,
                      float amplitude, const int* __restrict__ tok_pos) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ __align__(16) unsigned char hr_raw[];
  const int pitch = K + 8;
  __nv_bfloat16* xs = (__nv_bfloat16*)hr_raw;  // [16][pitch]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int h = blockIdx.y;
  const __nv_bfloat16* Ah = A + (size_t)h * lda_h;
  for (int c = tid; c < 16 * (K / 8); c += HR_WARPS * 32) {
    const int r = c / (K / 8), kc = (c - r * (K / 8)) * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < M) v = ldg16(Ah + (size_t)r * lda + kc);
    *(uint4*)(xs + r * pitch + kc) = v;
  }
  __syncthreads();
  if (tail > 0 && blockIdx.x == 0) {
    const int half = rot_dims >> 1;
    for (int e = tid; e < M * tail; e += HR_WARPS * 32) {
      const int r = e / tail, i = e % tail;
      const __nv_bfloat16* src = Ah + (size_t)r * lda + K;
      float v = __bfloat162float(src[i]);
      if (i < rot_dims) {
        const int f = i < half ? i : i - half;
        float sn, cs;
        sincosf(inv_freq[f] * (float)tok_pos[r], &sn, &cs);
        sn *= amplitude;
        cs *= amplitude;
        const float other = __bfloat162float(src[i < half ? i + half : i - half]);
        v = i < half ? v * cs - other * sn : v * cs + other * sn;
      }
      C[(size_t)r * ldc + (size_t)h * ldc_h + N + i] = __float2bfloat16_rn(v);
    }
  }
  const int n0 = (blockIdx.x * HR_WARPS + warp) * 16;
  if (n0 >= N) return;
  const __nv_bfloat16* Bh = B + (size_t)h * N * K;
  const __nv_bfloat16* wa = Bh + (size_t)min(n0 + g, N - 1) * K + 8 * t;      // rows past N: read
  const __nv_bfloat16* wb = Bh + (size_t)min(n0 + g + 8, N - 1) * K + 8 * t;  // again, not stored
  const __nv_bfloat16* x0 = xs + g * pitch + 8 * t;
  const __nv_bfloat16* x1 = x0 + 8 * pitch;
  float acc[2][4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  constexpr int UNROLL = 4;
  for (int k0 = 0; k0 < K; k0 += 32 * UNROLL) {
    uint4 a[UNROLL], b[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = k0 + 32 * u;
      if (k < K) {
        a[u] = ldg16(wa + k);
        b[u] = ldg16(wb + k);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = k0 + 32 * u;
      if (k < K) {
        const uint4 xa = *(const uint4*)(x0 + k), xb = *(const uint4*)(x1 + k);
        mma_bf16(acc[0], a[u].x, b[u].x, a[u].y, b[u].y, xa.x, xa.y);
        mma_bf16(acc[0], a[u].z, b[u].z, a[u].w, b[u].w, xa.z, xa.w);
        mma_bf16(acc[1], a[u].x, b[u].x, a[u].y, b[u].y, xb.x, xb.y);
        mma_bf16(acc[1], a[u].z, b[u].z, a[u].w, b[u].w, xb.z, xb.w);
      }
    }
  }
  // acc[nt][0..1]: feature n0 + g, tokens 8 nt + 2t and + 1; acc[nt][2..3]: feature n0 + g + 8
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int el = 0; el < 4; ++el) {
      const int gn = n0 + g + (el >= 2 ? 8 : 0), r = 8 * nt + 2 * t + (el & 1);
      if (gn >= N || r >= M) continue;
      float v = acc[nt][el];
      if (gate) {
        const float gv = __bfloat162float(gate[(size_t)r * ldg + (size_t)h * N + gn]);
        v *= 1.0f / (1.0f + expf(-gv));
      }
      C[(size_t)r * ldc + (size_t)h * ldc_h + gn] = __float2bfloat16_rn(v);
    }
}

MB_EXPORT int mb_heads_gemm(const void* A, int dtype, int lda, int lda_h, const void* B,
                            int b_dtype, void* C, int ldc, int ldc_h, int M, int N, int K,
                            int heads, const void* gate, int ldg, int tail, int rot_dims,
                            const float* inv_freq, float amplitude, const int* tok_pos,
                            void* stream) {
  if (M <= 0 || heads <= 0) return 0;
  if (tail > HG_BK * 20) MB_FAIL("mb_heads_gemm: a tail of %d values", tail);
  if (tail > 0 && (rot_dims > tail || (rot_dims & 1) || (rot_dims > 0 && !inv_freq) || !tok_pos))
    MB_FAIL("mb_heads_gemm: %d rotating values of a tail of %d", rot_dims, tail);
  cudaStream_t s = (cudaStream_t)stream;
  // bfloat16 operands whose rows start on 16-byte boundaries go to the tensor cores: up to 16
  // tokens (a decode step) to the form with the weight rows in the product's registers, more
  // to 128 x 128 tiles
  const bool aligned = dtype == MB_BF16 && b_dtype == MB_BF16 && K % 8 == 0 && lda % 8 == 0 &&
                       lda_h % 8 == 0 && (((uintptr_t)A | (uintptr_t)B) & 15) == 0;
  if (aligned && M <= 16 && K % 32 == 0 && (size_t)16 * (K + 8) * 2 <= 96 * 1024) {
    const size_t smem = (size_t)16 * (K + 8) * 2;
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(heads_rows_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           96 * 1024);
      configured = true;
    }
    mb_launch(heads_rows_mma_kernel, dim3((N + 16 * HR_WARPS - 1) / (16 * HR_WARPS), heads),
              dim3(HR_WARPS * 32), smem, s, (const __nv_bfloat16*)A, lda, lda_h,
              (const __nv_bfloat16*)B, (__nv_bfloat16*)C, ldc, ldc_h, M, N, K,
              (const __nv_bfloat16*)gate, ldg, tail, rot_dims, inv_freq, amplitude, tok_pos);
    MB_CHECK_LAUNCH("mb_heads_gemm");
  }
  if (aligned && M > 16) {
    mb_launch(heads_gemm_mma_kernel, dim3((N + 127) / 128, (M + MT_BM - 1) / MT_BM, heads),
              dim3(MT_THREADS), 0, s, (const __nv_bfloat16*)A, lda, lda_h, (const __nv_bfloat16*)B,
              (__nv_bfloat16*)C, ldc, ldc_h, M, N, K, (const __nv_bfloat16*)gate, ldg, tail,
              rot_dims, inv_freq, amplitude, tok_pos);
    MB_CHECK_LAUNCH("mb_heads_gemm");
  }
#define GO(T_, TB_, BM_)                                                                     \
  mb_launch(heads_gemm_kernel<T_, TB_, BM_>, dim3((N + HG_BN - 1) / HG_BN, (M + BM_ - 1) / BM_, \
                                                  heads),                                    \
            dim3(256), 0, s, (const T_*)A, lda, lda_h, (const TB_*)B, (T_*)C, ldc, ldc_h, M, N, \
            K, (const T_*)gate, ldg, tail, rot_dims, inv_freq, amplitude, tok_pos)
#define GO2(T_, TB_) \
  if (M <= 16) GO(T_, TB_, 16); else GO(T_, TB_, 64)
  if (dtype == MB_F32) {
    if (b_dtype == MB_F32) { GO2(float, float); } else { GO2(float, __nv_bfloat16); }
  } else {
    if (b_dtype == MB_F32) { GO2(__nv_bfloat16, float); } else { GO2(__nv_bfloat16, __nv_bfloat16); }
  }
#undef GO2
#undef GO
  MB_CHECK_LAUNCH("mb_heads_gemm");
}

// ------------------------------------------------------------------ latent_attention
// One block per (token, four heads): the block stages 32 rows of the cache [c ; r] in shared
// memory once, every warp (one head) scores its query against them (a lane a key), softmax
// on-line in float32, and adds p · c into its accumulators (the first kv_rank values of the
// same rows are the values). q [T, heads, dk] with dk = kv_rank + rot_dim; out [T, heads,
// kv_rank]. window > 0: only the last `window` positions are seen.
#define LAT_WARPS 4
#define LAT_MAX_D 32  // kv_rank up to 32 * LAT_MAX_D
template <typename T, bool VEC>
__global__ void __launch_bounds__(LAT_WARPS * 32)
latent_attention_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                        const T* __restrict__ pool, const int* __restrict__ page_table,
                        int max_pages, int ring_pages, const int* __restrict__ tok_slot,
                        const int* __restrict__ tok_pos, int nh, int kv_rank, int dk, int window,
                        float scale) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ __align__(16) float sm[];
  const int pitch = VEC ? dk + 4 : dk + 1;
  float* qs = sm;                      // [LAT_WARPS][dk]
  float* ks = qs + LAT_WARPS * dk;     // [32][pitch]
  __shared__ size_t rows[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * LAT_WARPS + warp;
  const bool live = h < nh;
  const int pos = tok_pos[t];
  const int slot = tok_slot[t];
  float* qv = qs + warp * dk;
  if (live) {
    const T* qp = q + (size_t)t * q_stride + (size_t)h * dk;
    for (int i = lane; i < dk; i += 32) qv[i] = to_f32<T>(qp[i]);
  }
  int lo = 0;
  if (window > 0 && pos + 1 > window) lo = pos + 1 - window;
  float m = -INFINITY, l = 0.f;
  float acc[LAT_MAX_D];
#pragma unroll
  for (int d = 0; d < LAT_MAX_D; ++d) acc[d] = 0.f;

  for (int k0 = lo; k0 <= pos; k0 += 32) {
    const int n = min(32, pos - k0 + 1);
    __syncthreads();  // the tile before has been read
    if (threadIdx.x < n)
      rows[threadIdx.x] = kv_row(page_table, max_pages, ring_pages, slot, k0 + threadIdx.x, 1, 0);
    __syncthreads();
    if (VEC) {
      const int pieces = dk / 4;
      for (int e = threadIdx.x; e < n * pieces; e += LAT_WARPS * 32) {
        const int key = e / pieces, piece = e - key * pieces;
        *(float4*)(ks + key * pitch + 4 * piece) = load4<T>(pool + rows[key] * dk + 4 * piece);
      }
    } else {
      for (int e = threadIdx.x; e < n * dk; e += LAT_WARPS * 32) {
        const int key = e / dk, i = e - key * dk;
        ks[key * pitch + i] = to_f32<T>(pool[rows[key] * dk + i]);
      }
    }
    __syncthreads();
    if (!live) continue;
    const bool valid = lane < n;
    float s = -INFINITY;
    if (valid) {
      const float* kr = ks + lane * pitch;
      float dot = 0.f;
      if (VEC) {
        for (int i = 0; i < dk; i += 4) {
          const float4 kk = *(const float4*)(kr + i), qq = *(const float4*)(qv + i);
          dot = fmaf(qq.x, kk.x, fmaf(qq.y, kk.y, fmaf(qq.z, kk.z, fmaf(qq.w, kk.w, dot))));
        }
      } else {
        for (int i = 0; i < dk; ++i) dot = fmaf(qv[i], kr[i], dot);
      }
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);  // 0 on the first tile (m = -inf)
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int d = 0; d < LAT_MAX_D; ++d) acc[d] *= corr;
    m = m_new;
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const float* vr = ks + j * pitch;
      if (VEC) {
#pragma unroll
        for (int d = 0; d < LAT_MAX_D / 4; ++d) {
          const int i = 4 * lane + 128 * d;
          if (i < kv_rank) {
            const float4 vv = *(const float4*)(vr + i);
            acc[4 * d] = fmaf(pj, vv.x, acc[4 * d]);
            acc[4 * d + 1] = fmaf(pj, vv.y, acc[4 * d + 1]);
            acc[4 * d + 2] = fmaf(pj, vv.z, acc[4 * d + 2]);
            acc[4 * d + 3] = fmaf(pj, vv.w, acc[4 * d + 3]);
          }
        }
      } else {
#pragma unroll
        for (int d = 0; d < LAT_MAX_D; ++d) {
          const int i = lane + 32 * d;
          if (i < kv_rank) acc[d] = fmaf(pj, vr[i], acc[d]);
        }
      }
    }
  }
  if (!live) return;
  const float inv = 1.0f / l;
  T* op = out + (size_t)t * out_stride + (size_t)h * kv_rank;
  if (VEC) {
#pragma unroll
    for (int d = 0; d < LAT_MAX_D / 4; ++d) {
      const int i = 4 * lane + 128 * d;
      if (i < kv_rank)
        store4<T>(op + i, make_float4(acc[4 * d] * inv, acc[4 * d + 1] * inv, acc[4 * d + 2] * inv,
                                      acc[4 * d + 3] * inv));
    }
  } else {
#pragma unroll
    for (int d = 0; d < LAT_MAX_D; ++d) {
      const int i = lane + 32 * d;
      if (i < kv_rank) op[i] = from_f32<T>(acc[d] * inv);
    }
  }
}

MB_EXPORT int mb_latent_attention(const void* q, int q_stride, void* out, int out_stride,
                                  const void* pool, int dtype, const int* page_table,
                                  int max_pages, int ring_pages, const int* tok_slot,
                                  const int* tok_pos, int T, int nh, int kv_rank, int rot_dim,
                                  int window, float scale, void* stream) {
  if (T <= 0) return 0;
  const int dk = kv_rank + rot_dim;
  if (kv_rank <= 0 || kv_rank > 32 * LAT_MAX_D)
    MB_FAIL("mb_latent_attention: a latent of %d values is not supported (at most %d)", kv_rank,
            32 * LAT_MAX_D);
  cudaStream_t s = (cudaStream_t)stream;
  const int four = dtype == MB_F32 ? 15 : 7;
  const bool vec = dk % 4 == 0 && kv_rank % 4 == 0 && out_stride % 4 == 0 &&
                   (((uintptr_t)out | (uintptr_t)pool) & four) == 0;
  const size_t smem = ((size_t)LAT_WARPS * dk + 32 * (size_t)(dk + (vec ? 4 : 1))) * sizeof(float);
  if (smem > 200 * 1024) MB_FAIL("mb_latent_attention: cache rows of %d values", dk);
  dim3 grid(T, (nh + LAT_WARPS - 1) / LAT_WARPS);
#define GO(T_, V_)                                                                            \
  {                                                                                           \
    static bool configured = false;                                                           \
    if (!configured) {                                                                        \
      cudaFuncSetAttribute(latent_attention_kernel<T_, V_>,                                   \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);          \
      configured = true;                                                                      \
    }                                                                                         \
    mb_launch(latent_attention_kernel<T_, V_>, grid, dim3(LAT_WARPS * 32), smem, s,           \
              (const T_*)q, q_stride, (T_*)out, out_stride, (const T_*)pool, page_table,      \
              max_pages, ring_pages, tok_slot, tok_pos, nh, kv_rank, dk, window, scale);      \
  }
  if (dtype == MB_F32) {
    if (vec) GO(float, true) else GO(float, false)
  } else {
    if (vec) GO(__nv_bfloat16, true) else GO(__nv_bfloat16, false)
  }
#undef GO
  MB_CHECK_LAUNCH("mb_latent_attention");
}
