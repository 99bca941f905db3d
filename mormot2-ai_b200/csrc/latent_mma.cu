// Latent attention on the warp-level tensor cores (m16n8k16, bfloat16 in, float32 scores,
// softmax and sums), for prefill and decode alike. The cache holds one row per token, the
// key/value latent c (kv_rank values) followed by the rotated key part that all heads share
// (rot_dim values); a query row has the same dk = kv_rank + rot_dim values (its plain part
// already carried into the latent space), and the result of a head is the weighted sum of the
// rows' first kv_rank values.
//
// Every head reads the SAME rows, so the rows of the score matrix are (token, head) pairs: a
// block takes 64 of them of one sequence, head fastest (a decode step's token with up to 64
// heads, or 64 / heads tokens of a prompt), streams the sequence's cache rows through shared
// memory 32 keys at a time (two stages of 16-byte cp.async, through the page table) and uses
// each tile for all of its rows. Eight warps: four groups of 16 rows x two halves. The two
// warps of a group each score 16 of a tile's 32 keys over all dk values (S = Q Kᵀ), agree on
// the rows' new maximum through shared memory, write their half of P = exp(S - max) there as
// bfloat16, and then each adds P · V for its half of the kv_rank output columns (V = the same
// tile, read with ldmatrix.trans), with the output rows in registers (kv_rank / 4 floats a
// thread). A decode step of few sequences deals the key tiles of a sequence out over `splits`
// blocks that leave (max, sum, unnormalised output) in float32 scratch; the block that
// finishes last (a ticket counter, no waiting) adds them up.
//
// Sizes: dk and kv_rank multiples of 16, kv_rank at most 512; other sizes use the kernel of
// latent.cu. There is no wait on another block or on a barrier object, so nothing can hang.
#include "mma_common.cuh"

MB_DEFINE_LAST_ERROR

#define LM_ROWS 64
#define LM_KEYS 32
#define LM_THREADS 256

__device__ __forceinline__ void lm_cp16(void* smem, const void* global, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(global), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void lm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}

__device__ __forceinline__ void lm_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}

// NV: the most n8 tiles of output columns a warp holds (kv_rank / 16 of them are used).
template <int NV>
__global__ void __launch_bounds__(LM_THREADS, 1)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                            __nv_bfloat16* __restrict__ out, int out_stride,
                            const __nv_bfloat16* __restrict__ pool,
                            const int* __restrict__ page_table, int max_pages, int ring_pages,
                            const int* __restrict__ seq_start, const int* __restrict__ seq_past,
                            const int* __restrict__ seq_slot, int B, int nh, int kv_rank, int dk,
                            int window, float scale, int splits, float* __restrict__ scratch,
                            unsigned int* __restrict__ tickets) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int pitch = dk + 8;  // bfloat16 per shared row of Q and K
  __nv_bfloat16* qs = (__nv_bfloat16*)smem_raw;                  // [64][pitch]
  __nv_bfloat16* ks = qs + LM_ROWS * pitch;                      // [2][32][pitch]
  __nv_bfloat16* ps = ks + 2 * LM_KEYS * pitch;                  // [4][16][40]
  float* mx = (float*)(ps + 4 * 16 * 40);                        // [4][2][16]
  int* row_pos = (int*)(mx + 4 * 2 * 16);                        // [64] position, -1: no row
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rg = warp >> 1, cs = warp & 1, g = lane >> 2, t = lane & 3;

  // which sequence, and which 64 of its (token, head) rows
  int b = 0, tile = blockIdx.x;
  for (; b < B; ++b) {
    const int tiles = ((seq_start[b + 1] - seq_start[b]) * nh + LM_ROWS - 1) / LM_ROWS;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (b >= B) return;
  const int first = seq_start[b], n_new = seq_start[b + 1] - first, past = seq_past[b];
  const int slot = seq_slot[b], split = blockIdx.y;
  const int row0 = tile * LM_ROWS;
  if (tid < LM_ROWS) {
    const int tok = (row0 + tid) / nh;
    row_pos[tid] = tok < n_new ? past + tok : -1;
  }
  // the rows' queries
  const int chunks = dk / 8;
  for (int c = tid; c < LM_ROWS * chunks; c += LM_THREADS) {
    const int r = c / chunks, kc = (c - r * chunks) * 8;
    const int tok = (row0 + r) / nh, head = (row0 + r) - tok * nh;
    const bool ok = tok < n_new;
    lm_cp16(qs + r * pitch + kc,
            ok ? q + (size_t)(first + tok) * q_stride + (size_t)head * dk + kc : q, ok);
  }
  asm volatile("cp.async.commit_group;\n" ::: "memory");
  const int tok_lo = row0 / nh, tok_hi = min(n_new - 1, (row0 + LM_ROWS - 1) / nh);
  const int key_hi = past + tok_hi;                               // the last key any row sees
  int key_lo = 0;
  if (window > 0) key_lo = max(0, past + tok_lo + 1 - window);
  const int tile_lo = key_lo / LM_KEYS, n_tiles = key_hi / LM_KEYS + 1 - tile_lo;

  // eight threads bring one key's row: a thread looks its key's page up once a tile and then
  // copies every eighth 16-byte piece of the row
  const int my_key = tid >> 3, my_piece = tid & 7;
  auto load_keys = [&](int stage, int j) {
    const int key = (tile_lo + j) * LM_KEYS + my_key;
    const bool ok = key <= key_hi;
    const size_t row = ok ? kv_row(page_table, max_pages, ring_pages, slot, key, 1, 0) : 0;
    const __nv_bfloat16* src = pool + row * dk;
    __nv_bfloat16* dst = ks + (stage * LM_KEYS + my_key) * pitch;
    for (int kc = my_piece * 8; kc < dk; kc += 64) lm_cp16(dst + kc, src + kc, ok);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  float o[NV][4];
#pragma unroll
  for (int i = 0; i < NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // rows g and g + 8
  const int nv = kv_rank / 16;             // n8 tiles of this warp's half of the columns
  const int col0 = cs * (kv_rank / 2);

  int j = split;
  if (j < n_tiles) load_keys(0, j);
  __syncthreads();                         // row_pos is visible
  const int pos_a = row_pos[16 * rg + g], pos_b = row_pos[16 * rg + g + 8];
  const int lo_a = window > 0 ? max(0, pos_a + 1 - window) : 0;
  const int lo_b = window > 0 ? max(0, pos_b + 1 - window) : 0;
  int stage = 0;
  for (; j < n_tiles; j += splits, stage ^= 1) {
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();                       // the tile (and, the first time, Q) is in place; the
                                           // tile before has been used by everyone
    if (j + splits < n_tiles) load_keys(stage ^ 1, j + splits);
    const __nv_bfloat16* kt = ks + stage * LM_KEYS * pitch;
    // ---- S = Q Kᵀ for this warp's 16 rows and its 16 of the tile's keys
    float s[2][4];
#pragma unroll
    for (int ni = 0; ni < 2; ++ni) s[ni][0] = s[ni][1] = s[ni][2] = s[ni][3] = 0.f;
    // four 8 x 8 pieces with one instruction each: of Q rows 0-7 / 8-15 x values k.. / k+8..
    // (the A operand), of K keys 0-7 x values k.. / k+8.., keys 8-15 x the same (the B
    // operands of the warp's two groups of eight keys)
    const __nv_bfloat16* qa = qs + (16 * rg + (lane & 15)) * pitch + (lane >> 4) * 8;
    const __nv_bfloat16* kb = kt + (16 * cs + (lane & 7) + ((lane >> 4) << 3)) * pitch +
                              ((lane >> 3) & 1) * 8;
    // two k steps at a time into accumulators of their own: four independent chains of
    // products instead of two (a chain's next product waits for the one before)
    float s2[2][4];
#pragma unroll
    for (int ni = 0; ni < 2; ++ni) s2[ni][0] = s2[ni][1] = s2[ni][2] = s2[ni][3] = 0.f;
    int k = 0;
#pragma unroll 2
    for (; k + 32 <= dk; k += 32) {
      uint32_t a[4], bq[4], a2[4], bq2[4];
      lm_ldmatrix_x4(a, qa + k);
      lm_ldmatrix_x4(bq, kb + k);
      lm_ldmatrix_x4(a2, qa + k + 16);
      lm_ldmatrix_x4(bq2, kb + k + 16);
      mma_bf16(s[0], a[0], a[1], a[2], a[3], bq[0], bq[1]);
      mma_bf16(s[1], a[0], a[1], a[2], a[3], bq[2], bq[3]);
      mma_bf16(s2[0], a2[0], a2[1], a2[2], a2[3], bq2[0], bq2[1]);
      mma_bf16(s2[1], a2[0], a2[1], a2[2], a2[3], bq2[2], bq2[3]);
    }
    if (k < dk) {
      uint32_t a[4], bq[4];
      lm_ldmatrix_x4(a, qa + k);
      lm_ldmatrix_x4(bq, kb + k);
      mma_bf16(s[0], a[0], a[1], a[2], a[3], bq[0], bq[1]);
      mma_bf16(s[1], a[0], a[1], a[2], a[3], bq[2], bq[3]);
    }
#pragma unroll
    for (int ni = 0; ni < 2; ++ni)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[ni][e] += s2[ni][e];
    // ---- scale, mask, the rows' maxima over this warp's keys
    const int key0 = (tile_lo + j) * LM_KEYS + 16 * cs + 2 * t;
    float mt[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int ni = 0; ni < 2; ++ni)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + 8 * ni + (e & 1);
        const bool seen = e < 2 ? (key <= pos_a && key >= lo_a) : (key <= pos_b && key >= lo_b);
        s[ni][e] = seen ? s[ni][e] * scale : -INFINITY;
        mt[e >> 1] = fmaxf(mt[e >> 1], s[ni][e]);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mt[r] = fmaxf(mt[r], __shfl_xor_sync(0xffffffffu, mt[r], 1));
      mt[r] = fmaxf(mt[r], __shfl_xor_sync(0xffffffffu, mt[r], 2));
    }
    if (t == 0) {
      mx[(rg * 2 + cs) * 16 + g] = mt[0];
      mx[(rg * 2 + cs) * 16 + g + 8] = mt[1];
    }
    __syncthreads();
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float other = mx[(rg * 2 + (cs ^ 1)) * 16 + g + 8 * r];
      const float m_new = fmaxf(m_run[r], fmaxf(mt[r], other));
      corr[r] = m_run[r] == -INFINITY ? 0.f : expf(m_run[r] - m_new);
      m_run[r] = m_new;
    }
    // ---- P = exp(S - max): this warp's half into shared memory, its sums kept here
    float sum[2] = {0.f, 0.f};
    __nv_bfloat16* pw = ps + (rg * 16 + g) * 40 + 16 * cs + 2 * t;
#pragma unroll
    for (int ni = 0; ni < 2; ++ni) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p[e] = s[ni][e] == -INFINITY ? 0.f : expf(s[ni][e] - m_run[e >> 1]);
        // the sum takes what the product will take: the value rounded to bfloat16
        p[e] = __bfloat162float(__float2bfloat16_rn(p[e]));
        sum[e >> 1] += p[e];
      }
      *(uint32_t*)(pw + 8 * ni) = pack_bf16(p[0], p[1]);
      *(uint32_t*)(pw + 8 * 40 + 8 * ni) = pack_bf16(p[2], p[3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + sum[r];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    __syncthreads();
    // ---- O += P V for this warp's half of the columns
    uint32_t pa[2][4];
    const __nv_bfloat16* pr = ps + (rg * 16 + g) * 40 + 2 * t;
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      pa[kk][0] = *(const uint32_t*)(pr + 16 * kk);
      pa[kk][1] = *(const uint32_t*)(pr + 8 * 40 + 16 * kk);
      pa[kk][2] = *(const uint32_t*)(pr + 16 * kk + 8);
      pa[kk][3] = *(const uint32_t*)(pr + 8 * 40 + 16 * kk + 8);
    }
    const __nv_bfloat16* vrow = kt + lane * pitch + col0;   // lane i names key i of the tile
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (i < nv) {
        uint32_t vb[4];
        lm_ldmatrix_x4_trans(vb, vrow + 8 * i);
        mma_bf16(o[i], pa[0][0], pa[0][1], pa[0][2], pa[0][3], vb[0], vb[1]);
        mma_bf16(o[i], pa[1][0], pa[1][1], pa[1][2], pa[1][3], vb[2], vb[3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  // ---- the rows' sums: within the four lanes of a row, then with the other half's warp
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  __syncthreads();
  if (t == 0) {
    mx[(rg * 2 + cs) * 16 + g] = l_run[0];
    mx[(rg * 2 + cs) * 16 + g + 8] = l_run[1];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row0 + 16 * rg + g + 8 * r;
    const int tok = row / nh, head = row - tok * nh;
    if (tok >= n_new) continue;
    const float l = l_run[r] + mx[(rg * 2 + (cs ^ 1)) * 16 + g + 8 * r];
    if (splits == 1) {
      const float inv = 1.0f / l;
      __nv_bfloat16* dst = out + (size_t)(first + tok) * out_stride + (size_t)head * kv_rank + col0;
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (i < nv)
          *(uint32_t*)(dst + 8 * i + 2 * t) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    } else {
      float* dst = scratch + ((size_t)((first + tok) * nh + head) * splits + split) * (kv_rank + 2);
      if (cs == 0 && t == 0) {
        dst[0] = m_run[r];
        dst[1] = l;
      }
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (i < nv) {
          dst[2 + col0 + 8 * i + 2 * t] = o[i][2 * r];
          dst[2 + col0 + 8 * i + 2 * t + 1] = o[i][2 * r + 1];
        }
    }
  }
  if (splits == 1) return;
  // ---- the block that finishes last of a tile's splits adds them up: out[row] =
  // sum_s exp(m_s - M) O_s / sum_s exp(m_s - M) l_s. The ticket counter wraps to 0 by itself,
  // so the next launch finds it as this one did; nobody waits for anybody.
  __shared__ unsigned int ticket;
  __threadfence();
  __syncthreads();
  if (tid == 0) ticket = atomicInc(&tickets[blockIdx.x], (unsigned)splits - 1);
  __syncthreads();
  if (ticket != (unsigned)splits - 1) return;
  __threadfence();
  const int width = kv_rank + 2;
  // every row's weights exp(m_s - M) / sum first (a thread a row), then all threads add the
  // splits' outputs up, a pair of columns each, with the splits' loads in flight together
  float* wts = (float*)ks;                                   // [64][16]
  const int rows_here = min(LM_ROWS, n_new * nh - row0);
  if (tid < rows_here) {
    const int row = row0 + tid;
    const float* src = scratch + ((size_t)first * nh + row) * splits * width;
    float m[16], l[16], M = -INFINITY;
#pragma unroll
    for (int sp = 0; sp < 16; ++sp) {
      m[sp] = sp < splits ? __ldcg(src + (size_t)sp * width) : -INFINITY;
      l[sp] = sp < splits ? __ldcg(src + (size_t)sp * width + 1) : 0.f;
      M = fmaxf(M, m[sp]);
    }
    float total = 0.f;
#pragma unroll
    for (int sp = 0; sp < 16; ++sp) {
      m[sp] = m[sp] == -INFINITY ? 0.f : expf(m[sp] - M);
      total = fmaf(m[sp], l[sp], total);
    }
    const float inv = 1.0f / total;
#pragma unroll
    for (int sp = 0; sp < 16; ++sp) wts[tid * 16 + sp] = m[sp] * inv;
  }
  __syncthreads();
  const int pairs = kv_rank / 2;
  for (int e = tid; e < rows_here * pairs; e += LM_THREADS) {
    const int r = e / pairs, c = 2 * (e - r * pairs);
    const int row = row0 + r;
    const float* src = scratch + ((size_t)first * nh + row) * splits * width + 2 + c;
    float2 part[16];
#pragma unroll
    for (int sp = 0; sp < 16; ++sp)
      part[sp] = sp < splits ? __ldcg((const float2*)(src + (size_t)sp * width))
                             : make_float2(0.f, 0.f);
    float v0 = 0.f, v1 = 0.f;
#pragma unroll
    for (int sp = 0; sp < 16; ++sp) {
      const float w = wts[r * 16 + sp];
      v0 = fmaf(w, part[sp].x, v0);
      v1 = fmaf(w, part[sp].y, v1);
    }
    const int tok = row / nh, head = row - tok * nh;
    *(uint32_t*)(out + (size_t)(first + tok) * out_stride + (size_t)head * kv_rank + c) =
        pack_bf16(v0, v1);
  }
}

// q [T, nh * dk] (row stride q_stride), out [T, nh * kv_rank]; `tiles` = the sum over the
// step's sequences of ceil(new tokens * nh / 64), as the host counts it; `splits` > 1 needs
// scratch of T * nh * splits * (kv_rank + 2) floats and `tickets`, `tiles` counters that are 0
// (the kernel leaves them 0).
MB_EXPORT int mb_latent_attention_mma(const void* q, int q_stride, void* out, int out_stride,
                                      const void* pool, const int* page_table, int max_pages,
                                      int ring_pages, const int* seq_start, const int* seq_past,
                                      const int* seq_slot, int B, int T, int tiles, int nh,
                                      int kv_rank, int rot_dim, int window, float scale,
                                      int splits, float* scratch, long long scratch_floats,
                                      unsigned int* tickets, void* stream) {
  if (T <= 0 || tiles <= 0) return 0;
  const int dk = kv_rank + rot_dim;
  if (dk % 16 || kv_rank % 16 || kv_rank > 512 || q_stride % 8 || out_stride % 2 ||
      (((uintptr_t)q | (uintptr_t)pool) & 15) || ((uintptr_t)out & 3))
    MB_FAIL("mb_latent_attention_mma: sizes %d + %d or alignment not supported", kv_rank, rot_dim);
  if (splits < 1) splits = 1;
  if (splits > 16) MB_FAIL("mb_latent_attention_mma: at most 16 splits, not %d", splits);
  if (splits > 1 && (scratch == nullptr || tickets == nullptr ||
                     (long long)T * nh * splits * (kv_rank + 2) > scratch_floats))
    MB_FAIL("mb_latent_attention_mma: scratch for %d splits", splits);
  cudaStream_t s = (cudaStream_t)stream;
  const int pitch = dk + 8;
  const size_t smem = ((size_t)LM_ROWS * pitch + 2 * LM_KEYS * pitch + 4 * 16 * 40) * 2 +
                      4 * 2 * 16 * sizeof(float) + LM_ROWS * sizeof(int);
  if (smem > 220 * 1024) MB_FAIL("mb_latent_attention_mma: cache rows of %d values", dk);
  dim3 grid(tiles, splits);
#define GO(NV_)                                                                               \
  {                                                                                           \
    static bool configured = false;                                                           \
    if (!configured) {                                                                        \
      cudaFuncSetAttribute(latent_attention_mma_kernel<NV_>,                                  \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);          \
      configured = true;                                                                      \
    }                                                                                         \
    mb_launch(latent_attention_mma_kernel<NV_>, grid, dim3(LM_THREADS), smem, s,              \
              (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,             \
              (const __nv_bfloat16*)pool, page_table, max_pages, ring_pages, seq_start,       \
              seq_past, seq_slot, B, nh, kv_rank, dk, window, scale, splits, scratch,         \
              tickets);                                                                       \
  }
  if (kv_rank <= 128) GO(8) else if (kv_rank <= 256) GO(16) else GO(32)
#undef GO
  MB_CHECK_LAUNCH("mb_latent_attention_mma");
}
