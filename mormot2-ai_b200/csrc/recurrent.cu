// Recurrent mixers: what runs token after token over a state of fixed size per sequence.
// The state lives in float32 in the engine's state arena ([slots][state_stride] floats; a
// mixer's part of a slot's row starts at `state_off`), is read when a step begins and written
// when it ends, so a sequence may be fed in portions of any size. Everything that enters a
// recurrence is float32: decays, gates, maxima, norms. One block per (sequence, head) walks the
// step's tokens of its sequence in order, sixteen at a time staged in shared memory; a thread
// owns one value column of the head's matrix state, which is kept in shared memory.
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

// ------------------------------------------------------------------ decaying matrix state
// A block stages SCAN_CT tokens of its head's inputs in shared memory at once (all loads in
// flight together), walks them without a barrier between tokens (a thread reads the staged
// vectors and its own column of the state), and then norms the chunk's outputs a warp a token.
#define SCAN_CT 16

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
  extern __shared__ __align__(16) float wk_smem[];
  const int DD = (D * D + 3) & ~3;
  float* S = wk_smem;                        // [D][D], S[i * D + j]: key channel i, value channel j
  float4* vec = (float4*)(S + DD);           // [CT][D]: r, k, decay, u * k
  float* sv = (float*)(vec + SCAN_CT * D);   // [CT][D] v
  float* sg = sv + SCAN_CT * D;              // [CT][D] g
  float* so = sg + SCAN_CT * D;              // [CT][D] o
  const int b = blockIdx.x, hd = blockIdx.y, j = threadIdx.x;
  const int warp = j >> 5, lane = j & 31, warps = blockDim.x >> 5;
  const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
  float* st = state + (size_t)seq_slot[b] * state_stride + state_off;
  float* Sg = st + W + (size_t)hd * D * D;
  for (int e = j; e < D * D; e += blockDim.x) S[e] = Sg[e];
  const bool own = j < D;
  const int col = hd * D + j;
  const float w0j = own ? w0[col] : 0.f, uj = own ? u[col] : 0.f;
  for (int c0 = 0; c0 < n; c0 += SCAN_CT) {
    const int cn = min(SCAN_CT, n - c0);
    if (own) {
      for (int tt = 0; tt < cn; ++tt) {
        const size_t at = (size_t)(t0 + c0 + tt) * ld + col;
        const float kj = k[at];
        vec[tt * D + j] = make_float4(r[at], kj, expf(-expf(lw[at] + w0j)), uj * kj);
        sv[tt * D + j] = v[at];
        sg[tt * D + j] = g[at];
      }
    }
    __syncthreads();
    if (own) {
      for (int tt = 0; tt < cn; ++tt) {
        const float vj = sv[tt * D + j];
        const float4* x = vec + tt * D;
        float o = 0.f;
        for (int i = 0; i < D; ++i) {
          const float4 xi = x[i];
          const float s = S[i * D + j];
          o = fmaf(xi.x, fmaf(xi.w, vj, s), o);
          S[i * D + j] = fmaf(xi.z, s, xi.y * vj);
        }
        so[tt * D + j] = o;
      }
    }
    __syncthreads();
    for (int tt = warp; tt < cn; tt += warps) {
      float ss = 0.f;
      for (int i = lane; i < D; i += 32) ss = fmaf(so[tt * D + i], so[tt * D + i], ss);
      const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
      T* orow = out + (size_t)(t0 + c0 + tt) * H * D + hd * D;
      for (int i = lane; i < D; i += 32) {
        const float gi = sg[tt * D + i];
        orow[i] = from_f32<T>(so[tt * D + i] * inv * normw[hd * D + i] * (gi / (1.0f + expf(-gi))));
      }
    }
    __syncthreads();
  }
  for (int e = j; e < D * D; e += blockDim.x) Sg[e] = S[e];
  if (hd == 0 && n > 0)
    for (int c = j; c < W; c += blockDim.x) st[c] = to_f32<T>(h[(size_t)(t0 + n - 1) * W + c]);
}

static size_t wkv_smem_bytes(int D) {
  return ((size_t)((D * D + 3) & ~3) + (size_t)SCAN_CT * D * 7) * sizeof(float);
}

MB_EXPORT int mb_wkv_scan(const float* r, const float* k, const float* v, const float* lw,
                          const float* g, int ld, const float* w0, const float* u,
                          const float* normw, float eps, float* state, long long state_stride,
                          long long state_off, const void* h, int dtype, int W,
                          const int* seq_start, const int* seq_slot, void* out, int B, int H,
                          int D, void* stream) {
  if (B <= 0) return 0;
  const size_t smem = wkv_smem_bytes(D);
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
  extern __shared__ __align__(16) float ml_smem[];
  const int DD = (D * DV + 3) & ~3;
  float* S = ml_smem;                          // [D][DV]
  float2* qk = (float2*)(S + DD);              // [CT][D]: q (scaled), k
  float* sv = (float*)(qk + SCAN_CT * D);      // [CT][DV] v
  float* sg = sv + SCAN_CT * DV;               // [CT][DV] the output gate's logit
  float* snum = sg + SCAN_CT * DV;             // [CT][DV] S^T q
  float* snq = snum + SCAN_CT * DV;            // [CT][D] n_i q_i
  float* sab = snq + SCAN_CT * D;              // [CT][4]: the state's factor, the input's, e^(-m)
  const int b = blockIdx.x, hd = blockIdx.y, j = threadIdx.x;
  const int warp = j >> 5, lane = j & 31, warps = blockDim.x >> 5;
  const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
  float* st = state + (size_t)seq_slot[b] * state_stride + state_off +
              (size_t)hd * ((size_t)D * DV + D + 1);
  for (int e = j; e < D * DV; e += blockDim.x) S[e] = st[e];
  const bool own_k = j < D, own_v = j < DV;
  float nj = own_k ? st[(size_t)D * DV + j] : 0.f;
  float m = st[(size_t)D * DV + D];          // thread 0's copy is the one that counts
  const float bih = bi[hd], bfh = bf[hd];
  for (int c0 = 0; c0 < n; c0 += SCAN_CT) {
    const int cn = min(SCAN_CT, n - c0);
    for (int tt = 0; tt < cn; ++tt) {
      const float* zr = z + (size_t)(t0 + c0 + tt) * ld;
      if (own_k) qk[tt * D + j] = make_float2(zr[cq + hd * D + j] * q_scale, zr[ck + hd * D + j]);
      if (own_v) {
        sv[tt * DV + j] = zr[cv + hd * DV + j];
        sg[tt * DV + j] = zr[cg + hd * DV + j];
      }
    }
    if (j == 0) {
      // the gates and the running maximum, token after token
      for (int tt = 0; tt < cn; ++tt) {
        const float* zr = z + (size_t)(t0 + c0 + tt) * ld;
        const float gi = cap * tanhf((zr[ci + hd] + bih) / cap);
        const float gf = log_sigmoid(cap * tanhf((zr[cf + hd] + bfh) / cap));
        const float m_new = fmaxf(gf + m, gi);
        sab[tt * 4] = expf(gf + m - m_new);
        sab[tt * 4 + 1] = expf(gi - m_new);
        sab[tt * 4 + 2] = expf(-m_new);
        m = m_new;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float a = sab[tt * 4], bb = sab[tt * 4 + 1];
      if (own_k) {
        const float2 x = qk[tt * D + j];
        nj = fmaf(a, nj, bb * x.y);
        snq[tt * D + j] = nj * x.x;
      }
      if (own_v) {
        const float bv = bb * sv[tt * DV + j];
        const float2* x = qk + tt * D;
        float num = 0.f;
        for (int i = 0; i < D; ++i) {
          const float2 xi = x[i];
          const float s = fmaf(a, S[i * DV + j], xi.y * bv);
          S[i * DV + j] = s;
          num = fmaf(s, xi.x, num);
        }
        snum[tt * DV + j] = num;
      }
    }
    __syncthreads();
    for (int tt = warp; tt < cn; tt += warps) {
      float nq = 0.f, ss = 0.f;
      for (int i = lane; i < D; i += 32) nq += snq[tt * D + i];
      for (int i = lane; i < DV; i += 32) ss = fmaf(snum[tt * DV + i], snum[tt * DV + i], ss);
      nq = warp_sum(nq);
      ss = warp_sum(ss);
      const float den = fmaxf(fabsf(nq), sab[tt * 4 + 2]) + 1e-6f;
      const float inv = 1.0f / sqrtf(ss / (den * den) / (float)DV + eps);
      T* orow = out + (size_t)(t0 + c0 + tt) * H * DV + hd * DV;
      for (int i = lane; i < DV; i += 32) {
        const float gate = 1.0f / (1.0f + expf(-sg[tt * DV + i]));
        orow[i] = from_f32<T>(snum[tt * DV + i] / den * inv * normw[hd * DV + i] * gate);
      }
    }
    __syncthreads();
  }
  for (int e = j; e < D * DV; e += blockDim.x) st[e] = S[e];
  if (own_k) st[(size_t)D * DV + j] = nj;
  if (j == 0) st[(size_t)D * DV + D] = m;
}

static size_t mlstm_smem_bytes(int D, int DV) {
  return ((size_t)((D * DV + 3) & ~3) + (size_t)SCAN_CT * (3 * D + 3 * DV + 4)) * sizeof(float);
}

MB_EXPORT int mb_mlstm_scan(const float* z, int ld, int cq, int ck, int cv, int cg, int ci, int cf,
                            const float* bi, const float* bf, float cap, float q_scale,
                            const float* normw, float eps, float* state, long long state_stride,
                            long long state_off, const int* seq_start, const int* seq_slot,
                            void* out, int dtype, int B, int H, int D, int DV, void* stream) {
  if (B <= 0) return 0;
  const size_t smem = mlstm_smem_bytes(D, DV);
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
