// Recurrent mixers: what runs token after token over a state of fixed size per sequence.
// The state lives in float32 in the engine's state arena ([slots][state_stride] floats; a
// mixer's part of a slot's row starts at `state_off`), is read when a step begins and written
// when it ends, so a sequence may be fed in portions of any size. Everything that enters a
// recurrence is float32: decays, gates, maxima, norms. One block per (sequence, head) walks the
// step's tokens of its sequence in order; a thread owns one value column of the head's matrix
// state, which is kept in shared memory.
//
//   token_shift   mix_s[t] = h[t] + (h[t-1] - h[t]) mu_s   for several s at once; h[-1] of a
//                 sequence is kept in the state (zeros before the first token)
//   wkv_scan      decay w = exp(-exp(lw + w0)); o_t = (S + diag(u) k v^T)^T r;
//                 S <- diag(w) S + k v^T; then o / rms(o) * norm * silu(g) per head
//   mlstm_scan    log gates i = cap tanh((zi + bi)/cap), f = logsigmoid(cap tanh((zf + bf)/cap));
//                 m' = max(f + m, i); S <- e^(f+m-m') S + e^(i-m') k v^T; n likewise with k;
//                 o = S^T q / (max(|n.q|, e^(-m')) + 1e-6); then o / rms(o) * norm * sigmoid(g)
#include "common.cuh"

MB_DEFINE_LAST_ERROR

// ------------------------------------------------------------------ token shift
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ h, const float* __restrict__ state,
                                   size_t state_stride, size_t state_off,
                                   const int* __restrict__ tok_seq,
                                   const int* __restrict__ seq_start,
                                   const int* __restrict__ seq_slot, const float* __restrict__ mu,
                                   int n_mix, T* __restrict__ out, int Ttok, int W) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  const bool first = seq_start[b] == t;
  const float* prev_state = state + (size_t)seq_slot[b] * state_stride + state_off;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float hv = to_f32<T>(h[(size_t)t * W + c]);
    const float pv = first ? prev_state[c] : to_f32<T>(h[(size_t)(t - 1) * W + c]);
    const float d = pv - hv;
    for (int s = 0; s < n_mix; ++s)
      out[((size_t)s * Ttok + t) * W + c] = from_f32<T>(fmaf(d, mu[(size_t)s * W + c], hv));
  }
}

MB_EXPORT int mb_token_shift(const void* h, int dtype, const float* state, long long state_stride,
                             long long state_off, const int* tok_seq, const int* seq_start,
                             const int* seq_slot, const float* mu, int n_mix, void* out, int T,
                             int W, void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = W >= 1024 ? 256 : 128;
  if (dtype == MB_F32)
    mb_launch(token_shift_kernel<float>, dim3(T), dim3(threads), 0, s, (const float*)h, state,
              (size_t)state_stride, (size_t)state_off, tok_seq, seq_start, seq_slot, mu, n_mix,
              (float*)out, T, W);
  else
    mb_launch(token_shift_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, s,
              (const __nv_bfloat16*)h, state, (size_t)state_stride, (size_t)state_off, tok_seq,
              seq_start, seq_slot, mu, n_mix, (__nv_bfloat16*)out, T, W);
  MB_CHECK_LAUNCH("mb_token_shift");
}

// Two sums over the block at once; `red` holds 66 floats.
__device__ __forceinline__ float2 block_sum2(float a, float b, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();
  if (lane == 0) {
    red[warp] = a;
    red[33 + warp] = b;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    float ta = lane < nw ? red[lane] : 0.f, tb = lane < nw ? red[33 + lane] : 0.f;
    ta = warp_sum(ta);
    tb = warp_sum(tb);
    if (lane == 0) {
      red[32] = ta;
      red[65] = tb;
    }
  }
  __syncthreads();
  return make_float2(red[32], red[65]);
}

// ------------------------------------------------------------------ decaying matrix state
// r, k, v, lw, g: float32 [T, ld] each (head hd's values at column hd * D + i); w0, u, normw:
// float32 [H * D]. State of a slot: [W values of the last h | H x D x D]. out [T, H * D].
template <typename T>
__global__ void wkv_scan_kernel(const float* __restrict__ r, const float* __restrict__ k,
                                const float* __restrict__ v, const float* __restrict__ lw,
                                const float* __restrict__ g, int ld,
                                const float* __restrict__ w0, const float* __restrict__ u,
                                const float* __restrict__ normw, float eps,
                                float* __restrict__ state, size_t state_stride, size_t state_off,
                                const T* __restrict__ h, int W, const int* __restrict__ seq_start,
                                const int* __restrict__ seq_slot, T* __restrict__ out, int H,
                                int D) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ float wk_smem[];
  float* S = wk_smem;            // [D][D], S[i * D + j]: key channel i, value channel j
  float* sr = S + D * D;         // [D] r
  float* sk = sr + D;            // [D] k
  float* sw = sk + D;            // [D] decay
  float* su = sw + D;            // [D] u * k
  float* red = su + D;           // 33
  const int b = blockIdx.x, hd = blockIdx.y, j = threadIdx.x;
  const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
  float* st = state + (size_t)seq_slot[b] * state_stride + state_off;
  float* Sg = st + W + (size_t)hd * D * D;
  for (int e = j; e < D * D; e += blockDim.x) S[e] = Sg[e];
  const bool own = j < D;
  const int col = hd * D + j;
  const float w0j = own ? w0[col] : 0.f, uj = own ? u[col] : 0.f, nwj = own ? normw[col] : 0.f;
  __syncthreads();
  for (int t = t0; t < t0 + n; ++t) {
    const size_t at = (size_t)t * ld + col;
    float vj = 0.f, gj = 0.f;
    if (own) {
      const float kj = k[at];
      sr[j] = r[at];
      sk[j] = kj;
      sw[j] = expf(-expf(lw[at] + w0j));
      su[j] = uj * kj;
      vj = v[at];
      gj = g[at];
    }
    __syncthreads();
    float o = 0.f;
    if (own) {
      for (int i = 0; i < D; ++i) {
        const float s = S[i * D + j];
        o = fmaf(sr[i], fmaf(su[i], vj, s), o);
        S[i * D + j] = fmaf(sw[i], s, sk[i] * vj);
      }
    }
    const float ss = block_sum(own ? o * o : 0.f, red);   // also keeps the vectors' readers apart
    if (own) {
      const float inv = 1.0f / sqrtf(ss / (float)D + eps);
      const float gate = gj / (1.0f + expf(-gj));
      out[(size_t)t * H * D + col] = from_f32<T>(o * inv * nwj * gate);
    }
  }
  __syncthreads();
  for (int e = j; e < D * D; e += blockDim.x) Sg[e] = S[e];
  if (hd == 0 && n > 0)
    for (int c = j; c < W; c += blockDim.x) st[c] = to_f32<T>(h[(size_t)(t0 + n - 1) * W + c]);
}

MB_EXPORT int mb_wkv_scan(const float* r, const float* k, const float* v, const float* lw,
                          const float* g, int ld, const float* w0, const float* u,
                          const float* normw, float eps, float* state, long long state_stride,
                          long long state_off, const void* h, int dtype, int W,
                          const int* seq_start, const int* seq_slot, void* out, int B, int H,
                          int D, void* stream) {
  if (B <= 0) return 0;
  const size_t smem = ((size_t)D * D + 4 * D + 33) * sizeof(float);
  if (D <= 0 || D > 1024 || smem > 200 * 1024)
    MB_FAIL("mb_wkv_scan: heads of %d values (the state of a head must fit 200 KB)", D);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = (D + 31) / 32 * 32;
#define GO(T_)                                                                                 \
  {                                                                                            \
    static size_t configured = 48 * 1024;                                                      \
    if (smem > configured) {                                                                   \
      cudaFuncSetAttribute(wkv_scan_kernel<T_>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                           200 * 1024);                                                        \
      configured = 200 * 1024;                                                                 \
    }                                                                                          \
    mb_launch(wkv_scan_kernel<T_>, dim3(B, H), dim3(threads), smem, s, r, k, v, lw, g, ld, w0, \
              u, normw, eps, state, (size_t)state_stride, (size_t)state_off, (const T_*)h, W,  \
              seq_start, seq_slot, (T_*)out, H, D);                                            \
  }
  if (dtype == MB_F32) GO(float) else GO(__nv_bfloat16)
#undef GO
  MB_CHECK_LAUNCH("mb_wkv_scan");
}

// ------------------------------------------------------------------ matrix memory with gates
// z: float32 [T, ld], the fused projection: q at column cq + hd * D, k at ck + hd * D, v at
// cv + hd * DV, the output gate at cg + hd * DV, the input and forget gates at ci + hd and
// cf + hd. bi, bf: float32 [H]. normw: float32 [H * DV]. State of a slot, per head:
// [D x DV | D of n | m].
__device__ __forceinline__ float log_sigmoid(float x) {
  return fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
}

template <typename T>
__global__ void mlstm_scan_kernel(const float* __restrict__ z, int ld, int cq, int ck, int cv,
                                  int cg, int ci, int cf, const float* __restrict__ bi,
                                  const float* __restrict__ bf, float cap, float q_scale,
                                  const float* __restrict__ normw, float eps,
                                  float* __restrict__ state, size_t state_stride,
                                  size_t state_off, const int* __restrict__ seq_start,
                                  const int* __restrict__ seq_slot, T* __restrict__ out, int H,
                                  int D, int DV) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ float ml_smem[];
  float* S = ml_smem;          // [D][DV]
  float* sq = S + D * DV;      // [D]
  float* sk = sq + D;          // [D]
  float* sc = sk + D;          // a, b, exp(-m')
  float* red = sc + 4;         // 66
  const int b = blockIdx.x, hd = blockIdx.y, j = threadIdx.x;
  const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
  float* st = state + (size_t)seq_slot[b] * state_stride + state_off +
              (size_t)hd * ((size_t)D * DV + D + 1);
  for (int e = j; e < D * DV; e += blockDim.x) S[e] = st[e];
  const bool own_k = j < D, own_v = j < DV;
  float nj = own_k ? st[(size_t)D * DV + j] : 0.f;
  float m = st[(size_t)D * DV + D];
  const float bih = bi[hd], bfh = bf[hd];
  const float nwj = own_v ? normw[hd * DV + j] : 0.f;
  __syncthreads();
  for (int t = t0; t < t0 + n; ++t) {
    const float* zr = z + (size_t)t * ld;
    // every thread forms the gates itself (two values, the same arithmetic in each)
    const float gi = cap * tanhf((zr[ci + hd] + bih) / cap);
    const float gf = log_sigmoid(cap * tanhf((zr[cf + hd] + bfh) / cap));
    const float m_new = fmaxf(gf + m, gi);
    const float a = expf(gf + m - m_new), bb = expf(gi - m_new);
    m = m_new;
    float qj = 0.f, kj = 0.f, vj = 0.f, gj = 0.f;
    if (own_k) {
      qj = zr[cq + hd * D + j] * q_scale;
      kj = zr[ck + hd * D + j];
      sq[j] = qj;
      sk[j] = kj;
      nj = fmaf(a, nj, bb * kj);
    }
    if (own_v) {
      vj = zr[cv + hd * DV + j];
      gj = zr[cg + hd * DV + j];
    }
    __syncthreads();
    float num = 0.f;
    if (own_v) {
      const float bv = bb * vj;
      for (int i = 0; i < D; ++i) {
        const float s = fmaf(a, S[i * DV + j], sk[i] * bv);
        S[i * DV + j] = s;
        num = fmaf(s, sq[i], num);
      }
    }
    const float2 sums = block_sum2(own_k ? nj * qj : 0.f, own_v ? num * num : 0.f, red);
    if (own_v) {
      const float den = fmaxf(fabsf(sums.x), expf(-m)) + 1e-6f;
      const float inv = 1.0f / sqrtf(sums.y / (den * den) / (float)DV + eps);
      const float gate = 1.0f / (1.0f + expf(-gj));
      out[(size_t)t * H * DV + hd * DV + j] = from_f32<T>(num / den * inv * nwj * gate);
    }
  }
  __syncthreads();
  for (int e = j; e < D * DV; e += blockDim.x) st[e] = S[e];
  if (own_k) st[(size_t)D * DV + j] = nj;
  if (j == 0) st[(size_t)D * DV + D] = m;
}

MB_EXPORT int mb_mlstm_scan(const float* z, int ld, int cq, int ck, int cv, int cg, int ci, int cf,
                            const float* bi, const float* bf, float cap, float q_scale,
                            const float* normw, float eps, float* state, long long state_stride,
                            long long state_off, const int* seq_start, const int* seq_slot,
                            void* out, int dtype, int B, int H, int D, int DV, void* stream) {
  if (B <= 0) return 0;
  const size_t smem = ((size_t)D * DV + 2 * D + 4 + 66) * sizeof(float);
  if (D <= 0 || DV <= 0 || D > 1024 || DV > 1024 || smem > 200 * 1024)
    MB_FAIL("mb_mlstm_scan: heads of %d x %d values (the state of a head must fit 200 KB)", D, DV);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = ((D > DV ? D : DV) + 31) / 32 * 32;
#define GO(T_)                                                                                 \
  {                                                                                            \
    static size_t configured = 48 * 1024;                                                      \
    if (smem > configured) {                                                                   \
      cudaFuncSetAttribute(mlstm_scan_kernel<T_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           200 * 1024);                                                        \
      configured = 200 * 1024;                                                                 \
    }                                                                                          \
    mb_launch(mlstm_scan_kernel<T_>, dim3(B, H), dim3(threads), smem, s, z, ld, cq, ck, cv, cg, \
              ci, cf, bi, bf, cap, q_scale, normw, eps, state, (size_t)state_stride,           \
              (size_t)state_off, seq_start, seq_slot, (T_*)out, H, D, DV);                     \
  }
  if (dtype == MB_F32) GO(float) else GO(__nv_bfloat16)
#undef GO
  MB_CHECK_LAUNCH("mb_mlstm_scan");
}

// ------------------------------------------------------------------ tanh between two products
template <typename T>
__global__ void tanh_kernel(const float* __restrict__ in, T* __restrict__ out, size_t total) {
  mb_grid_wait();
  mb_grid_launch_next();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(tanhf(in[i]));
}

// out = tanh(in) for `total` float32 values, rounded to the activation type.
MB_EXPORT int mb_tanh(const float* in, void* out, int out_dtype, long long total, void* stream) {
  if (total <= 0) return 0;
  const long long want = (total + 255) / 256;
  const dim3 grid((unsigned)(want < 148 * 8 ? want : 148 * 8));
  if (out_dtype == MB_F32)
    mb_launch(tanh_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, in, (float*)out,
              (size_t)total);
  else
    mb_launch(tanh_kernel<__nv_bfloat16>, grid, dim3(256), 0, (cudaStream_t)stream, in,
              (__nv_bfloat16*)out, (size_t)total);
  MB_CHECK_LAUNCH("mb_tanh");
}
