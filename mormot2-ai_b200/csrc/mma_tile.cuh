// A 128-row output tile of C = A · Bᵀ on the warp-level tensor cores (m16n8k16, bfloat16 in,
// float32 accumulators), for products whose rows are gathered through pointers and whose
// weight is one of many small ones (a head's, an expert's): the batched and the grouped
// products of latent attention and of routed experts. The tile is 128 x 128 outputs, or, with
// NB = 2, 128 x 64 outputs of two weight blocks at once (a gate and an up projection of the
// same rows). Eight warps as 4 x 2, each 32 rows x half of the columns; K in steps of 32
// through two shared-memory stages filled with 16-byte cp.async (rows that do not exist and
// the tail of K are filled with zeros); fragments are read with ldmatrix.
//
// Every row of A and B must start on a 16-byte boundary and K must be a multiple of 8.
#pragma once
#include "mma_common.cuh"

#define MT_BM 128
#define MT_BK 32
#define MT_PITCH 40  // bfloat16 per shared row: 80 bytes, ldmatrix free of bank conflicts
#define MT_THREADS 256

template <int NB>
struct MtShared {
  static constexpr int BN = 128 / NB;  // output columns of the tile (per weight block)
  __nv_bfloat16 a[2][MT_BM][MT_PITCH];
  __nv_bfloat16 b[2][NB][BN][MT_PITCH];
  const __nv_bfloat16* a_rows[MT_BM];  // the tile's rows of A; null: a row of zeros
};

__device__ __forceinline__ void mt_cp16(void* smem, const void* global, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: nothing is read, 16 zero bytes are written
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(global), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mt_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}

// acc[nb][mi][ni][4]: warp (wm, wn) holds rows 32 wm + 16 mi + {g, g + 8} and columns
// (BN / 2) wn + 8 ni + {2t, 2t + 1} (g = lane / 4, t = lane % 4) in the m16n8 accumulator
// order. b[nb] points at the tile's first weight row of block nb (row n at b[nb] + n * K);
// n_valid of the BN rows exist. sh.a_rows must be filled and visible before the call.
template <int NB>
__device__ __forceinline__ void mt_mainloop(MtShared<NB>& sh, const __nv_bfloat16* const* b,
                                            int n_valid, int K,
                                            float (&acc)[NB][2][8 / NB][4]) {
  constexpr int BN = 128 / NB, NI = 8 / NB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1;
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int ni = 0; ni < NI; ++ni)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nb][mi][ni][e] = 0.f;
  const int nk = (K + MT_BK - 1) / MT_BK;
  auto load = [&](int stage, int kt) {
    const int k0 = kt * MT_BK;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = tid + i * MT_THREADS;
      const int r = c >> 2, kc = (c & 3) * 8;
      const __nv_bfloat16* row = sh.a_rows[r];
      const bool ok = row != nullptr && k0 + kc < K;
      mt_cp16(&sh.a[stage][r][kc], ok ? row + k0 + kc : b[0], ok);
      // the same chunk index names a row of the weight: r of block 0, or r - BN of block 1
      const int nb = r / BN, rn = r - nb * BN;
      const bool okb = rn < n_valid && k0 + kc < K;
      mt_cp16(&sh.b[stage][nb][rn][kc], okb ? b[nb] + (size_t)rn * K + k0 + kc : b[0], okb);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  load(0, 0);
  for (int kt = 0; kt < nk; ++kt) {
    const int stage = kt & 1;
    if (kt + 1 < nk) {
      load(stage ^ 1, kt + 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < MT_BK; ks += 16) {
      // A: rows 0-7 / 8-15 of the 16 x values ks.. / ks+8.. as four 8 x 8 pieces
      uint32_t af[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
        mt_ldmatrix_x4(af[mi], &sh.a[stage][32 * wm + 16 * mi + (lane & 15)][ks + (lane >> 4) * 8]);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int np = 0; np < NI / 2; ++np) {
          // B: weight rows 0-7 x values ks.. / ks+8.., rows 8-15 x the same: two n8 tiles
          uint32_t bf[4];
          mt_ldmatrix_x4(bf, &sh.b[stage][nb][(BN / 2) * wn + 16 * np + (lane & 7) +
                                               ((lane >> 4) << 3)][ks + ((lane >> 3) & 1) * 8]);
#pragma unroll
          for (int mi = 0; mi < 2; ++mi) {
            mma_bf16(acc[nb][mi][2 * np], af[mi][0], af[mi][1], af[mi][2], af[mi][3], bf[0], bf[1]);
            mma_bf16(acc[nb][mi][2 * np + 1], af[mi][0], af[mi][1], af[mi][2], af[mi][3], bf[2],
                     bf[3]);
          }
        }
    }
    __syncthreads();
  }
}

// Calls f(row, col, mi, ni, e) for every accumulator element of this thread: row within the
// tile's 128 rows, col within its BN columns; the value is acc[nb][mi][ni][e].
template <int NB, typename F>
__device__ __forceinline__ void mt_for_each(F f) {
  constexpr int BN = 128 / NB, NI = 8 / NB;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wm = warp >> 1, wn = warp & 1, g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int ni = 0; ni < NI; ++ni)
#pragma unroll
      for (int e = 0; e < 4; ++e)
        f(32 * wm + 16 * mi + g + (e >= 2 ? 8 : 0), (BN / 2) * wn + 8 * ni + 2 * t + (e & 1), mi,
          ni, e);
}
