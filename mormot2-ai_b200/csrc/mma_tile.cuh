// A 64 x 64 output tile of C = A · Bᵀ on the warp-level tensor cores (m16n8k16, bfloat16 in,
// float32 accumulators), for products whose rows are gathered through pointers and whose
// weight is one of many small ones (a head's, an expert's): the batched and the grouped
// products of latent attention and of routed experts. Four warps as 2 x 2, each 32 x 32 of the
// tile; K in steps of 32 through two shared-memory stages filled with 16-byte cp.async (rows
// that do not exist and the tail of K are filled with zeros). NB = 2 multiplies the same rows
// with two weight blocks at once (a gate and an up projection).
//
// Every row of A and B must start on a 16-byte boundary and K must be a multiple of 8.
#pragma once
#include "mma_common.cuh"

#define MT_BM 64
#define MT_BN 64
#define MT_BK 32
#define MT_PITCH 40  // bfloat16 per shared row: 80 bytes, fragment reads free of bank conflicts

template <int NB>
struct MtShared {
  __nv_bfloat16 a[2][MT_BM][MT_PITCH];
  __nv_bfloat16 b[2][NB][MT_BN][MT_PITCH];
  const __nv_bfloat16* a_rows[MT_BM];  // the tile's rows of A; null: a row of zeros
};

__device__ __forceinline__ void mt_cp16(void* smem, const void* global, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: nothing is read, 16 zero bytes are written
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(global), "r"(bytes)
               : "memory");
}

// acc[nb][mi][ni][4]: warp (wm, wn) holds rows 32 wm + 16 mi + {g, g + 8} and columns
// 32 wn + 8 ni + {2t, 2t + 1} (g = lane / 4, t = lane % 4) in the m16n8 accumulator order.
// b[nb] points at the tile's first weight row of block nb (row n at b[nb] + n * K); n_valid of
// the 64 rows exist. sh.a_rows must be filled and visible (a __syncthreads) before the call.
template <int NB>
__device__ __forceinline__ void mt_mainloop(MtShared<NB>& sh, const __nv_bfloat16* const* b,
                                            int n_valid, int K, float (&acc)[NB][2][4][4]) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1, g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int ni = 0; ni < 4; ++ni)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nb][mi][ni][e] = 0.f;
  const int nk = (K + MT_BK - 1) / MT_BK;
  auto load = [&](int stage, int kt) {
    const int k0 = kt * MT_BK;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = tid + i * 128;
      const int r = c >> 2, kc = (c & 3) * 8;
      const __nv_bfloat16* row = sh.a_rows[r];
      const bool ok = row != nullptr && k0 + kc < K;
      mt_cp16(&sh.a[stage][r][kc], ok ? row + k0 + kc : b[0], ok);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const bool okb = r < n_valid && k0 + kc < K;
        mt_cp16(&sh.b[stage][nb][r][kc], okb ? b[nb] + (size_t)r * K + k0 + kc : b[0], okb);
      }
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
      uint32_t af[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) {
        const __nv_bfloat16* p = &sh.a[stage][32 * wm + 16 * mi + g][ks + 2 * t];
        af[mi][0] = *(const uint32_t*)p;
        af[mi][1] = *(const uint32_t*)(p + 8 * MT_PITCH);
        af[mi][2] = *(const uint32_t*)(p + 8);
        af[mi][3] = *(const uint32_t*)(p + 8 * MT_PITCH + 8);
      }
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) {
          const __nv_bfloat16* p = &sh.b[stage][nb][32 * wn + 8 * ni + g][ks + 2 * t];
          const uint32_t b0 = *(const uint32_t*)p, b1 = *(const uint32_t*)(p + 8);
#pragma unroll
          for (int mi = 0; mi < 2; ++mi)
            mma_bf16(acc[nb][mi][ni], af[mi][0], af[mi][1], af[mi][2], af[mi][3], b0, b1);
        }
    }
    __syncthreads();
  }
}

// Calls f(row, col, e) for every accumulator element e of this thread: row and col within
// the 64 x 64 tile; the value is acc[nb][mi][ni][e] with (mi, ni, e) as f receives them.
template <typename F>
__device__ __forceinline__ void mt_for_each(F f) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wm = warp >> 1, wn = warp & 1, g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int ni = 0; ni < 4; ++ni)
#pragma unroll
      for (int e = 0; e < 4; ++e)
        f(32 * wm + 16 * mi + g + (e >= 2 ? 8 : 0), 32 * wn + 8 * ni + 2 * t + (e & 1), mi, ni, e);
}
