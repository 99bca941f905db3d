// A feed-forward of routed experts on the device, without a round trip to the host: the
// router's choice, the lists of tokens per expert, the experts' two products over those lists
// and the weighted sum into the residual. float32 arithmetic on the CUDA cores for float32
// and bfloat16 storage.
//
//   moe_route    per token: the `top` largest router logits (the lower index on a tie), their
//                weights = softmax over the chosen logits only, and the shared expert's gate
//                sigmoid(logit) when the router's product carries that column
//   moe_plan     assignments (token, k) listed expert by expert, cut into tiles of rows
//   moe_gemm     for every tile the product with its expert's weight:
//                up:   act[r, :] = f(h[token(r)] · Wgᵀ) * (h[token(r)] · Wuᵀ)   (rows gathered)
//                down: y[a(r), :] = weight[a(r)] * (act[r] · Wdᵀ)              (float32, scattered
//                      to the assignment's own row, so the sum below has a fixed order)
//   moe_combine  x[t] += sum_k y[t·top + k] + gate[t] · shared[t]
//
// The order of an expert's rows in its list comes from atomic counters and may differ from run
// to run; no result depends on it (a row's sums are formed alone, in a fixed order).
#include "common.cuh"
#include "mma_tile.cuh"

MB_DEFINE_LAST_ERROR

// ------------------------------------------------------------------ route
// z [parts][T, ldz] float32, the split sums of the router's product (parts = 1: the product
// itself), added up as they are read: columns [0, E) the experts' logits, column shared_col
// (or -1) the shared expert's gate logit. One warp per token.
__device__ __forceinline__ float route_logit(const float* __restrict__ zr, int parts,
                                             size_t part_stride, int i) {
  return parts == 1 ? zr[i] : sum_parts(zr + i, parts, part_stride);
}

__device__ __forceinline__ void route_token(const float* __restrict__ zr, int parts,
                                            size_t part_stride, int E, int top, int shared_col,
                                            int* __restrict__ ids, float* __restrict__ w,
                                            float* __restrict__ sg, int lane) {
  float last_v = INFINITY;
  int last_i = -1;
  float first = 0.f, sum = 0.f, mine = 0.f;  // lane k keeps the k-th chosen logit
  // up to 256 experts: a lane adds its logits' split sums up once and keeps them
  const bool kept = E <= 256;
  float zl[8];
  if (kept) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = lane + 32 * j;
      zl[j] = i < E ? route_logit(zr, parts, part_stride, i) : -INFINITY;
    }
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    if (kept) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = lane + 32 * j;
        const float v = zl[j];
        const bool open = i < E && (v < last_v || (v == last_v && i > last_i));
        if (open && (v > best || (v == best && i < best_i))) {
          best = v;
          best_i = i;
        }
      }
    } else {
      for (int i = lane; i < E; i += 32) {
        const float v = route_logit(zr, parts, part_stride, i);
        const bool open = v < last_v || (v == last_v && i > last_i);
        if (open && (v > best || (v == best && i < best_i))) {
          best = v;
          best_i = i;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (best_i == 0x7fffffff) {  // nothing left that compares (NaNs): take the next index
      best_i = min(E - 1, last_i + 1);
      best = route_logit(zr, parts, part_stride, best_i);
    }
    if (k == 0) first = best;
    const float e = expf(best - first);
    sum += e;
    if (lane == k) mine = e;
    if (lane == 0) ids[k] = best_i;
    last_v = best;
    last_i = best_i;
  }
  if (lane < top) w[lane] = mine / sum;
  if (sg && lane == 0) *sg = 1.0f / (1.0f + expf(-route_logit(zr, parts, part_stride, shared_col)));
}

// The other scoring: s = softmax(z) over all E columns; the choice goes by s + corr (the lower
// index on a tie), the weights are the chosen s times wscale, not renormalized. Up to 256
// columns (a lane keeps eight).
__device__ __forceinline__ void route_token_scored(const float* __restrict__ zr, int parts,
                                                   size_t part_stride, int E, int top,
                                                   const float* __restrict__ corr, float wscale,
                                                   int* __restrict__ ids, float* __restrict__ w,
                                                   int lane) {
  float sc[8], ch[8];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = lane + 32 * j;
    sc[j] = i < E ? route_logit(zr, parts, part_stride, i) : -INFINITY;
    mx = fmaxf(mx, sc[j]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    sc[j] = lane + 32 * j < E ? expf(sc[j] - mx) : 0.f;
    sum += sc[j];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = lane + 32 * j;
    sc[j] = sc[j] / sum;
    ch[j] = i < E ? sc[j] + (corr ? corr[i] : 0.f) : -INFINITY;
  }
  float last_v = INFINITY, mine = 0.f;
  int last_i = -1;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY, best_s = 0.f;
    int best_i = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = lane + 32 * j;
      const float v = ch[j];
      const bool open = i < E && (v < last_v || (v == last_v && i > last_i));
      if (open && (v > best || (v == best && i < best_i))) {
        best = v;
        best_i = i;
        best_s = sc[j];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
        best_s = os;
      }
    }
    if (best_i == 0x7fffffff) {  // nothing left that compares (NaNs): take the next index
      best_i = min(E - 1, last_i + 1);
      best_s = 0.f;
    }
    if (lane == k) mine = best_s * wscale;
    if (lane == 0) ids[k] = best_i;
    last_v = best;
    last_i = best_i;
  }
  if (lane < top) w[lane] = mine;
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ z, int ldz, int parts, size_t part_stride, int E,
                 int top, int shared_col, int* __restrict__ ids, float* __restrict__ w,
                 float* __restrict__ sg, int T, int mode, const float* __restrict__ corr,
                 float wscale) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  if (mode == 1) {
    route_token_scored(z + (size_t)t * ldz, parts, part_stride, E, top, corr, wscale,
                       ids + (size_t)t * top, w + (size_t)t * top, lane);
    return;
  }
  route_token(z + (size_t)t * ldz, parts, part_stride, E, top, shared_col, ids + (size_t)t * top,
              w + (size_t)t * top, sg ? sg + t : nullptr, lane);
}

MB_EXPORT int mb_moe_route(const float* z, int ldz, int parts, long long part_stride, int E,
                           int top, int shared_col, int* ids, float* w, float* sg, int T,
                           int mode, const float* corr, float wscale, void* stream) {
  if (T <= 0) return 0;
  if (mode == 1 && (E > 256 || sg != nullptr))
    MB_FAIL("mb_moe_route: scores over all of %d columns (at most 256, no gate column)", E);
  if (top <= 0 || top > 32 || top > E) MB_FAIL("mb_moe_route: %d of %d experts", top, E);
  if ((sg != nullptr) != (shared_col >= 0)) MB_FAIL("mb_moe_route: the shared gate and its column");
  if (parts < 1) MB_FAIL("mb_moe_route: %d parts", parts);
  mb_launch(moe_route_kernel, dim3((T + 3) / 4), dim3(128), 0, (cudaStream_t)stream, z, ldz,
            parts, (size_t)part_stride, E, top, shared_col, ids, w, sg, T, mode, corr, wscale);
  MB_CHECK_LAUNCH("mb_moe_route");
}

// ------------------------------------------------------------------ plan
// plan (int32): [0] number of tiles, [1 .. 1+E] first list row of every expert (E + 1 values),
// then perm[A] (the assignment a = t·top + k at every list row), then tile_expert[max_tiles]
// and tile_row0[max_tiles]. One block.
// With z given (a step of at most 64 tokens) the block first routes the tokens itself, a warp a
// token, and writes ids, w and sg as moe_route does: one kernel instead of two.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(int* __restrict__ ids, int A, int E, int bm, int max_tiles,
                int* __restrict__ plan, const float* __restrict__ z, int ldz, int parts,
                size_t part_stride, int top, int shared_col, float* __restrict__ w,
                float* __restrict__ sg, int mode, const float* __restrict__ corr, float wscale,
                int E_route) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ int counts[];  // E counters, then E cursors
  if (z != nullptr) {
    const int T = A / top, lane = threadIdx.x & 31;
    for (int t = threadIdx.x >> 5; t < T; t += blockDim.x >> 5) {
      if (mode == 1)
        route_token_scored(z + (size_t)t * ldz, parts, part_stride, E_route, top, corr, wscale,
                           ids + (size_t)t * top, w + (size_t)t * top, lane);
      else
        route_token(z + (size_t)t * ldz, parts, part_stride, E_route, top, shared_col,
                    ids + (size_t)t * top, w + (size_t)t * top, sg ? sg + t : nullptr, lane);
    }
    __syncthreads();  // the block's own writes of ids are visible to it
  }
  int* cursor = counts + E;
  int* offsets = plan + 1;
  int* perm = offsets + E + 1;
  int* tile_e = perm + A;
  int* tile_r0 = tile_e + max_tiles;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int a = threadIdx.x; a < A; a += blockDim.x) {
    const int e = ids[a];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      cursor[e] = at;
      for (int r0 = 0; r0 < counts[e] && tiles < max_tiles; r0 += bm) {
        tile_e[tiles] = e;
        tile_r0[tiles] = at + r0;
        ++tiles;
      }
      at += counts[e];
    }
    offsets[E] = at;
    plan[0] = tiles;
  }
  __syncthreads();
  for (int a = threadIdx.x; a < A; a += blockDim.x) {
    const int e = ids[a];
    if (e >= 0 && e < E) perm[atomicAdd(&cursor[e], 1)] = a;
  }
}

MB_EXPORT int mb_moe_plan(int* ids, int A, int E, int bm, int max_tiles, int* plan,
                          void* stream) {
  if (A <= 0) return 0;
  if (E > 4096) MB_FAIL("mb_moe_plan: %d experts", E);
  if (max_tiles < (A + bm - 1) / bm + E) MB_FAIL("mb_moe_plan: room for %d tiles", max_tiles);
  mb_launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int),
            (cudaStream_t)stream, ids, A, E, bm, max_tiles, plan, (const float*)nullptr, 0, 1,
            (size_t)0, 1, -1, (float*)nullptr, (float*)nullptr, 0, (const float*)nullptr, 1.0f, E);
  MB_CHECK_LAUNCH("mb_moe_plan");
}

// moe_route and moe_plan in one kernel, for a step of at most 64 tokens.
MB_EXPORT int mb_moe_route_plan(const float* z, int ldz, int parts, long long part_stride, int E,
                                int top, int shared_col, int* ids, float* w, float* sg, int T,
                                int bm, int max_tiles, int* plan, int mode, const float* corr,
                                float wscale, int E_route, void* stream) {
  if (T <= 0) return 0;
  if (E_route < E) MB_FAIL("mb_moe_route_plan: %d routed columns for %d experts", E_route, E);
  if (mode == 1 && (E_route > 256 || sg != nullptr))
    MB_FAIL("mb_moe_route_plan: scores over all of %d columns (at most 256, no gate column)", E_route);
  if (T > 64) MB_FAIL("mb_moe_route_plan: %d tokens (at most 64)", T);
  if (top <= 0 || top > 32 || top > E_route) MB_FAIL("mb_moe_route_plan: %d of %d experts", top, E_route);
  if ((sg != nullptr) != (shared_col >= 0)) MB_FAIL("mb_moe_route_plan: the shared gate and its column");
  if (E > 4096 || parts < 1) MB_FAIL("mb_moe_route_plan: %d experts, %d parts", E, parts);
  const int A = T * top;
  if (max_tiles < (A + bm - 1) / bm + E) MB_FAIL("mb_moe_route_plan: room for %d tiles", max_tiles);
  mb_launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int),
            (cudaStream_t)stream, ids, A, E, bm, max_tiles, plan, z, ldz, parts,
            (size_t)part_stride, top, shared_col, w, sg, mode, corr, wscale, E_route);
  MB_CHECK_LAUNCH("mb_moe_route_plan");
}

// ------------------------------------------------------------------ the experts' products
// act(gate) * up. 0: SiLU; 1: the tanh form of GELU; 2: the clamped form
// g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(1.702 g') (u' + 1).
__device__ __forceinline__ float moe_gated(float z, float u, int act, float limit) {
  if (act == 2) {
    z = fminf(z, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return z / (1.0f + expf(-1.702f * z)) * (u + 1.0f);
  }
  if (act == 1)
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))) * u;
  return z / (1.0f + expf(-z)) * u;
}

#define MG_BN 64
#define MG_BK 16
// UP:   in = h [T, K] (row of list row r: perm[r] / top), W [E][2N][K] (gate rows, then up
//       rows), out = act [A, N] at list row r.
// DOWN: in = act [A, K] at list row r, W [E][N][K], out = y [A, N] float32 at row perm[r],
//       multiplied by weight[perm[r]].
template <typename T, typename TW, int BM, bool UP>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ in, const TW* __restrict__ W, void* __restrict__ out,
                const int* __restrict__ plan, int A, int E, int max_tiles, int top, int N, int K,
                int act, const float* __restrict__ weight, float limit) {
  mb_grid_wait();
  mb_grid_launch_next();
  constexpr int NW = UP ? 2 : 1;
  constexpr int TM = BM / 16;
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int* offsets = plan + 1;
  const int* perm = offsets + E + 1;
  const int e = perm[A + tile];
  const int r0 = perm[A + max_tiles + tile];
  const int rows = min(BM, offsets[e + 1] - r0);
  __shared__ float As[MG_BK][BM + 4];
  __shared__ float Ws[NW][MG_BK][MG_BN + 4];
  __shared__ int src[BM];
  const int tid = threadIdx.x;
  if (tid < BM) src[tid] = tid < rows ? perm[r0 + tid] : -1;
  __syncthreads();
  const int n0 = blockIdx.x * MG_BN;
  const TW* We = W + (size_t)e * NW * N * K;
  const int tr = (tid / 16) * TM, tc = (tid % 16) * 4;
  float acc[NW][TM][4];
#pragma unroll
  for (int w = 0; w < NW; ++w)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[w][i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += MG_BK) {
    for (int el = tid; el < BM * MG_BK; el += 256) {
      const int r = el / MG_BK, c = el % MG_BK;
      const int gk = k0 + c;
      float v = 0.f;
      if (r < rows && gk < K) {
        const size_t row = UP ? (size_t)(src[r] / top) : (size_t)(r0 + r);
        v = to_f32<T>(in[row * K + gk]);
      }
      As[c][r] = v;
    }
    for (int el = tid; el < MG_BN * MG_BK; el += 256) {
      const int r = el / MG_BK, c = el % MG_BK;
      const int gn = n0 + r, gk = k0 + c;
#pragma unroll
      for (int w = 0; w < NW; ++w)
        Ws[w][c][r] = (gn < N && gk < K) ? to_f32<TW>(We[((size_t)w * N + gn) * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MG_BK; ++k) {
      float a[TM];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][tr + i];
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        float b[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Ws[w][k][tc + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[w][i][j] = fmaf(a[i], b[j], acc[w][i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = tr + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tc + j;
      if (gn >= N) continue;
      if (UP) {
        ((T*)out)[(size_t)(r0 + r) * N + gn] =
            from_f32<T>(moe_gated(acc[0][i][j], acc[NW - 1][i][j], act, limit));
      } else {
        const int a = src[r];
        ((float*)out)[(size_t)a * N + gn] = weight[a] * acc[0][i][j];
      }
    }
  }
}

// The same two products on the tensor cores for bfloat16 operands (mma_tile.cuh); the plan's
// tiles have 128 rows. The first product multiplies the gathered rows with the gate and the up
// rows of the expert at once.
template <bool UP>
__global__ void __launch_bounds__(MT_THREADS)
moe_gemm_mma_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ W,
                    void* __restrict__ out, const int* __restrict__ plan, int A, int E,
                    int max_tiles, int top, int N, int K, int act,
                    const float* __restrict__ weight, float limit) {
  mb_grid_wait();
  mb_grid_launch_next();
  constexpr int NB = UP ? 2 : 1;
  constexpr int MT_BN = 128 / NB;
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int* offsets = plan + 1;
  const int* perm = offsets + E + 1;
  const int e = perm[A + tile];
  const int r0 = perm[A + max_tiles + tile];
  const int rows = min(MT_BM, offsets[e + 1] - r0);
  __shared__ __align__(16) MtShared<NB> sh;
  __shared__ int src[MT_BM];
  if (threadIdx.x < MT_BM) {
    const int r = threadIdx.x;
    const int a = r < rows ? perm[r0 + r] : -1;
    src[r] = a;
    sh.a_rows[r] = a < 0 ? nullptr : in + (UP ? (size_t)(a / top) : (size_t)(r0 + r)) * K;
  }
  __syncthreads();
  const int n0 = blockIdx.x * MT_BN;
  const __nv_bfloat16* We = W + (size_t)e * NB * N * K;
  const __nv_bfloat16* b[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) b[nb] = We + ((size_t)nb * N + n0) * K;
  float acc[NB][2][8 / NB][4];
  mt_mainloop<NB>(sh, b, min(MT_BN, N - n0), K, acc);
  mt_for_each<NB>([&](int r, int c, int mi, int ni, int el) {
    const int gn = n0 + c;
    if (r >= rows || gn >= N) return;
    if (UP) {
      ((__nv_bfloat16*)out)[(size_t)(r0 + r) * N + gn] =
          __float2bfloat16_rn(moe_gated(acc[0][mi][ni][el], acc[NB - 1][mi][ni][el], act, limit));
    } else {
      const int a = src[r];
      ((float*)out)[(size_t)a * N + gn] = weight[a] * acc[0][mi][ni][el];
    }
  });
}

// The two products for a decode step of at most eight tokens (tiles of at most 8 rows, so an
// expert's weights are streamed exactly once): the WEIGHT rows are the 16 rows of the m16n8k16
// product and the tile's tokens its 8 columns. A warp owns 16 output features (for the first
// product their gate and their up rows) over all of K and reads its weight rows straight from
// global memory into the product's registers, 16 bytes a thread and row, several steps of K in
// flight; the tokens' rows wait in shared memory. Within a step of 32 values of K a thread
// holds values 8t .. 8t+7 of both operands: the products pair them up in another order than
// the instruction's own, which is the same sum. K must be a multiple of 32.
#define MR_WARPS 4
template <bool UP>
__global__ void __launch_bounds__(MR_WARPS * 32)
moe_rows_mma_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ W,
                    void* __restrict__ out, const int* __restrict__ plan, int A, int E,
                    int max_tiles, int top, int N, int K, int act,
                    const float* __restrict__ weight, float limit) {
  mb_grid_wait();
  mb_grid_launch_next();
  constexpr int NB = UP ? 2 : 1;
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int* offsets = plan + 1;
  const int* perm = offsets + E + 1;
  const int e = perm[A + tile];
  const int r0 = perm[A + max_tiles + tile];
  const int rows = min(8, offsets[e + 1] - r0);
  extern __shared__ __align__(16) unsigned char mr_raw[];
  const int pitch = K + 8;
  __nv_bfloat16* xs = (__nv_bfloat16*)mr_raw;  // [8][pitch]
  __shared__ int src[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  if (tid < 8) src[tid] = tid < rows ? perm[r0 + tid] : -1;
  __syncthreads();
  for (int c = tid; c < 8 * (K / 8); c += MR_WARPS * 32) {
    const int r = c / (K / 8), kc = (c - r * (K / 8)) * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows) v = ldg16(in + (UP ? (size_t)(src[r] / top) : (size_t)(r0 + r)) * K + kc);
    *(uint4*)(xs + r * pitch + kc) = v;
  }
  __syncthreads();
  const int n0 = (blockIdx.x * MR_WARPS + warp) * 16;
  if (n0 >= N) return;
  const __nv_bfloat16* We = W + (size_t)e * NB * N * K;
  // rows past N are read from row N - 1 and never stored
  const __nv_bfloat16* wa[NB];
  const __nv_bfloat16* wb[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    wa[nb] = We + ((size_t)nb * N + min(n0 + g, N - 1)) * K + 8 * t;
    wb[nb] = We + ((size_t)nb * N + min(n0 + g + 8, N - 1)) * K + 8 * t;
  }
  const __nv_bfloat16* xr = xs + g * pitch + 8 * t;
  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;
  constexpr int UNROLL = UP ? 4 : 8;
  for (int k0 = 0; k0 < K; k0 += 32 * UNROLL) {
    uint4 a[UNROLL][NB], b[UNROLL][NB];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = k0 + 32 * u;
      if (k < K) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          a[u][nb] = ldg16(wa[nb] + k);
          b[u][nb] = ldg16(wb[nb] + k);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = k0 + 32 * u;
      if (k < K) {
        const uint4 x = *(const uint4*)(xr + k);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          mma_bf16(acc[nb], a[u][nb].x, b[u][nb].x, a[u][nb].y, b[u][nb].y, x.x, x.y);
          mma_bf16(acc[nb], a[u][nb].z, b[u][nb].z, a[u][nb].w, b[u][nb].w, x.z, x.w);
        }
      }
    }
  }
  // acc[.][0..1]: feature n0 + g, tokens 2t and 2t + 1; acc[.][2..3]: feature n0 + g + 8
#pragma unroll
  for (int el = 0; el < 4; ++el) {
    const int gn = n0 + g + (el >= 2 ? 8 : 0), r = 2 * t + (el & 1);
    if (gn >= N || r >= rows) continue;
    if (UP) {
      ((__nv_bfloat16*)out)[(size_t)(r0 + r) * N + gn] =
          __float2bfloat16_rn(moe_gated(acc[0][el], acc[NB - 1][el], act, limit));
    } else {
      const int a_ = src[r];
      ((float*)out)[(size_t)a_ * N + gn] = weight[a_] * acc[0][el];
    }
  }
}

MB_EXPORT int mb_moe_gemm(const void* in, int dtype, const void* W, int w_dtype, void* out,
                          const int* plan, int A, int E, int max_tiles, int bm, int top, int N,
                          int K, int up, int act, const float* weight, float limit, void* stream) {
  if (A <= 0) return 0;
  if (bm != 8 && bm != 16 && bm != 64 && bm != 128) MB_FAIL("mb_moe_gemm: tiles of %d rows", bm);
  if (!up && weight == nullptr) MB_FAIL("mb_moe_gemm: the second product needs the weights");
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid((N + MG_BN - 1) / MG_BN, max_tiles);
  if (bm == 8) {
    if (!(dtype == MB_BF16 && w_dtype == MB_BF16 && K % 32 == 0 &&
          (((uintptr_t)in | (uintptr_t)W) & 15) == 0))
      MB_FAIL("mb_moe_gemm: tiles of 8 rows are the decode kernel's (bfloat16, K %% 32 == 0)");
    const size_t smem = (size_t)8 * (K + 8) * 2;
    if (smem > 160 * 1024) MB_FAIL("mb_moe_gemm: rows of %d values", K);
    dim3 g8((N + 16 * MR_WARPS - 1) / (16 * MR_WARPS), max_tiles);
#define GO8(UP_)                                                                              \
  {                                                                                           \
    static bool configured = false;                                                           \
    if (!configured) {                                                                        \
      cudaFuncSetAttribute(moe_rows_mma_kernel<UP_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           160 * 1024);                                                       \
      configured = true;                                                                      \
    }                                                                                         \
    mb_launch(moe_rows_mma_kernel<UP_>, g8, dim3(MR_WARPS * 32), smem, s,                     \
              (const __nv_bfloat16*)in, (const __nv_bfloat16*)W, out, plan, A, E, max_tiles,  \
              top, N, K, act, weight, limit);                                                 \
  }
    if (up) GO8(true) else GO8(false)
#undef GO8
    MB_CHECK_LAUNCH("mb_moe_gemm");
  }
  if (bm == 128) {
    if (!(dtype == MB_BF16 && w_dtype == MB_BF16 && K % 8 == 0 &&
          (((uintptr_t)in | (uintptr_t)W) & 15) == 0))
      MB_FAIL("mb_moe_gemm: tiles of 128 rows are the tensor-core kernel's (bfloat16, K %% 8 == 0)");
    if (up)
      mb_launch(moe_gemm_mma_kernel<true>, dim3((N + 63) / 64, max_tiles), dim3(MT_THREADS), 0, s,
                (const __nv_bfloat16*)in, (const __nv_bfloat16*)W, out, plan, A, E, max_tiles, top,
                N, K, act, weight, limit);
    else
      mb_launch(moe_gemm_mma_kernel<false>, dim3((N + 127) / 128, max_tiles), dim3(MT_THREADS), 0,
                s, (const __nv_bfloat16*)in, (const __nv_bfloat16*)W, out, plan, A, E, max_tiles,
                top, N, K, act, weight, limit);
    MB_CHECK_LAUNCH("mb_moe_gemm");
  }
#define GO(T_, TW_, BM_, UP_)                                                                \
  mb_launch(moe_gemm_kernel<T_, TW_, BM_, UP_>, grid, dim3(256), 0, s, (const T_*)in,        \
            (const TW_*)W, out, plan, A, E, max_tiles, top, N, K, act, weight, limit)
#define GO3(T_, TW_)                                                  \
  {                                                                   \
    if (bm == 16) { if (up) GO(T_, TW_, 16, true); else GO(T_, TW_, 16, false); } \
    else { if (up) GO(T_, TW_, 64, true); else GO(T_, TW_, 64, false); }          \
  }
  if (dtype == MB_F32) {
    if (w_dtype == MB_F32) GO3(float, float) else GO3(float, __nv_bfloat16)
  } else {
    if (w_dtype == MB_F32) GO3(__nv_bfloat16, float) else GO3(__nv_bfloat16, __nv_bfloat16)
  }
#undef GO3
#undef GO
  MB_CHECK_LAUNCH("mb_moe_gemm");
}

// ------------------------------------------------------------------ combine
// x[t, c] += sum_k y[(t·top + k), c] (k ascending) + sg[t] · shared[t, c]; shared
// [parts][T, H]: the split sums of the shared expert's last product, added up in split order.
// An assignment whose expert id is E or more names an identity expert: its term is
// w[a] · h[t, c] (h: the feed-forward's input, `h_bf16` says of which type). `store`: x = the
// sum instead of x += it.
__global__ void moe_combine_kernel(float* __restrict__ x, const float* __restrict__ y, int top,
                                   const float* __restrict__ shared, int parts,
                                   size_t part_stride, const float* __restrict__ sg, int H,
                                   const int* __restrict__ ids, const float* __restrict__ w,
                                   int E, const void* __restrict__ h, int h_bf16, int store) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int t = blockIdx.x;
  const float g = sg ? sg[t] : 1.0f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < top; ++k) {
      const size_t a = (size_t)t * top + k;
      if (ids != nullptr && ids[a] >= E) {
        const float hv = h_bf16 ? __bfloat162float(((const __nv_bfloat16*)h)[(size_t)t * H + c])
                                : ((const float*)h)[(size_t)t * H + c];
        v = fmaf(w[a], hv, v);
      } else {
        v += y[a * H + c];
      }
    }
    if (shared) {
      v = fmaf(g, sum_parts(shared + (size_t)t * H + c, parts, part_stride), v);
    }
    if (store) x[(size_t)t * H + c] = v;
    else x[(size_t)t * H + c] += v;
  }
}

MB_EXPORT int mb_moe_combine(float* x, const float* y, int top, const float* shared, int parts,
                             long long part_stride, const float* sg, int T, int H,
                             const int* ids, const float* w, int E, const void* h, int h_dtype,
                             int store, void* stream) {
  if (T <= 0) return 0;
  if (ids != nullptr && (w == nullptr || h == nullptr))
    MB_FAIL("mb_moe_combine: identity experts need the weights and the input rows");
  mb_launch(moe_combine_kernel, dim3(T), dim3(H >= 1024 ? 256 : 128), 0, (cudaStream_t)stream, x,
            y, top, shared, parts, (size_t)part_stride, sg, H, ids, w, E, h,
            h_dtype == MB_BF16 ? 1 : 0, store);
  MB_CHECK_LAUNCH("mb_moe_combine");
}
