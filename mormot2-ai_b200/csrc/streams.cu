// Several residual streams (hyper-connections) and the layer norm that reads them.
//
// A model may keep S copies x_0 .. x_(S-1) of the residual [S][T, H] (float32). A sublayer
// reads u = sum_s in[s] x_s, normed, and its output y comes back into every stream at once:
//     x_t <- sum_s mix[s, t] x_s + out[t] y          (mix indexed [from, to])
// One kernel does the write-back of the sublayer before (y may be a sum of several terms with
// a factor each: the branches of a mixer that runs side by side) and the read for the next
// one, so the streams pass through memory once per sublayer. With S = 1, no write-back and
// in = 1 it is a plain layer norm of the residual; with `rows` it norms a gather of rows (the
// model's last norm over the rows whose logits are wanted).
//
// Layer norm: (u - mean) / sqrt(var + eps) * w, var the mean of the squared deviations (two
// passes over the row, which is kept in shared memory), no bias. Everything in float32.
#include "common.cuh"

MB_DEFINE_LAST_ERROR

#define ST_MAX_STREAMS 8
#define ST_MAX_TERMS 16

struct StTerms {
  const float* y[ST_MAX_TERMS];  // [T, H] float32 each
  float scale[ST_MAX_TERMS];
  int n;
};

__device__ __forceinline__ float4 f4_scale(float a, float4 v) {
  return make_float4(a * v.x, a * v.y, a * v.z, a * v.w);
}
__device__ __forceinline__ float4 f4_fma(float a, float4 v, float4 acc) {
  return make_float4(fmaf(a, v.x, acc.x), fmaf(a, v.y, acc.y), fmaf(a, v.z, acc.z),
                     fmaf(a, v.w, acc.w));
}

// V = 4: four neighbouring columns a thread and step (H a multiple of 4, every pointer on a
// 16-byte boundary); V = 1: one. The arithmetic of a column is the same in both.
template <typename TW, typename TO, int V>
__global__ void stream_step_kernel(float* __restrict__ x, size_t stream_stride, int S,
                                   const float* __restrict__ mix, const float* __restrict__ outc,
                                   StTerms terms, const float* __restrict__ in,
                                   const TW* __restrict__ w, float eps, TO* __restrict__ out,
                                   const int* __restrict__ rows, int H) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ __align__(16) float st_smem[];  // H values of u, then 33 for the reductions
  __shared__ float s_mix[ST_MAX_STREAMS * ST_MAX_STREAMS], s_out[ST_MAX_STREAMS],
      s_in[ST_MAX_STREAMS];
  float* u_row = st_smem;
  float* red = st_smem + H;
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  if (threadIdx.x < S * S) s_mix[threadIdx.x] = mix ? mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    s_out[threadIdx.x] = outc ? outc[threadIdx.x] : 0.f;
    s_in[threadIdx.x] = in ? in[threadIdx.x] : 1.f;
  }
  __syncthreads();
  float sum = 0.f;
  if (V == 4) {
    for (int c = 4 * threadIdx.x; c < H; c += 4 * blockDim.x) {
      float4 xs[ST_MAX_STREAMS];
#pragma unroll
      for (int s = 0; s < ST_MAX_STREAMS; ++s)
        xs[s] = s < S ? *(const float4*)(x + (size_t)s * stream_stride + (size_t)t * H + c)
                      : make_float4(0.f, 0.f, 0.f, 0.f);
      if (mix) {
        float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int b = 0; b < terms.n; ++b) {
          const float4 v = *(const float4*)(terms.y[b] + (size_t)t * H + c);
          y = b == 0 ? f4_scale(terms.scale[0], v) : f4_fma(terms.scale[b], v, y);
        }
        float4 nx[ST_MAX_STREAMS];
#pragma unroll
        for (int to = 0; to < ST_MAX_STREAMS; ++to) {
          if (to < S) {
            float4 v = f4_scale(s_out[to], y);
#pragma unroll
            for (int s = 0; s < ST_MAX_STREAMS; ++s)
              if (s < S) v = f4_fma(s_mix[s * S + to], xs[s], v);
            nx[to] = v;
            *(float4*)(x + (size_t)to * stream_stride + (size_t)t * H + c) = v;
          }
        }
#pragma unroll
        for (int s = 0; s < ST_MAX_STREAMS; ++s)
          if (s < S) xs[s] = nx[s];
      }
      if (w) {
        float4 u = f4_scale(s_in[0], xs[0]);
#pragma unroll
        for (int s = 1; s < ST_MAX_STREAMS; ++s)
          if (s < S) u = f4_fma(s_in[s], xs[s], u);
        *(float4*)(u_row + c) = u;
        sum += (u.x + u.y) + (u.z + u.w);
      }
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float xs[ST_MAX_STREAMS];
#pragma unroll
      for (int s = 0; s < ST_MAX_STREAMS; ++s)
        xs[s] = s < S ? x[(size_t)s * stream_stride + (size_t)t * H + c] : 0.f;
      if (mix) {
        float y = 0.f;
        for (int b = 0; b < terms.n; ++b) {
          const float v = terms.y[b][(size_t)t * H + c];
          y = b == 0 ? terms.scale[0] * v : fmaf(terms.scale[b], v, y);
        }
        float nx[ST_MAX_STREAMS];
#pragma unroll
        for (int to = 0; to < ST_MAX_STREAMS; ++to) {
          if (to < S) {
            float v = s_out[to] * y;
#pragma unroll
            for (int s = 0; s < ST_MAX_STREAMS; ++s)
              if (s < S) v = fmaf(s_mix[s * S + to], xs[s], v);
            nx[to] = v;
            x[(size_t)to * stream_stride + (size_t)t * H + c] = v;
          }
        }
#pragma unroll
        for (int s = 0; s < ST_MAX_STREAMS; ++s) xs[s] = s < S ? nx[s] : 0.f;
      }
      if (w) {
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < ST_MAX_STREAMS; ++s)
          if (s < S) u = s == 0 ? s_in[0] * xs[0] : fmaf(s_in[s], xs[s], u);
        u_row[c] = u;
        sum += u;
      }
    }
  }
  if (!w) return;
  const float mean = block_sum(sum, red) / (float)H;
  float dev = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float d = u_row[c] - mean;
    dev = fmaf(d, d, dev);
  }
  const float inv = 1.0f / sqrtf(block_sum(dev, red) / (float)H + eps);
  if (V == 4) {
    for (int c = 4 * threadIdx.x; c < H; c += 4 * blockDim.x) {
      const float4 u = *(const float4*)(u_row + c), ww = load4<TW>(w + c);
      store4<TO>(out + (size_t)r * H + c,
                 make_float4((u.x - mean) * inv * ww.x, (u.y - mean) * inv * ww.y,
                             (u.z - mean) * inv * ww.z, (u.w - mean) * inv * ww.w));
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x)
      out[(size_t)r * H + c] = from_f32<TO>((u_row[c] - mean) * inv * to_f32<TW>(w[c]));
  }
}

// x: [S][T, H] float32, stream s at x + s * stream_stride. mix [S, S], outc [S] and the terms:
// the write-back (mix null: none). in [S] (null: ones), w [H], out [R, H]: the read and its
// layer norm (w null: none). rows [R] or null (then R = T rows in order); a write-back
// together with rows is refused.
MB_EXPORT int mb_stream_step(float* x, long long stream_stride, int S, const float* mix,
                             const float* outc, const float* const* ys, const float* scales,
                             int n_terms, const float* in, const void* w, int w_dtype, float eps,
                             void* out, int out_dtype, const int* rows, int R, int H,
                             void* stream) {
  if (R <= 0) return 0;
  if (S < 1 || S > ST_MAX_STREAMS) MB_FAIL("mb_stream_step: %d streams (1 to %d)", S, ST_MAX_STREAMS);
  if (mix && rows) MB_FAIL("mb_stream_step: a write-back with a row gather");
  if (mix && (n_terms < 1 || n_terms > ST_MAX_TERMS || !outc))
    MB_FAIL("mb_stream_step: a write-back of %d terms (1 to %d)", n_terms, ST_MAX_TERMS);
  if (!mix && !w) return 0;
  StTerms terms;
  terms.n = mix ? n_terms : 0;
  for (int b = 0; b < ST_MAX_TERMS; ++b) {
    terms.y[b] = b < terms.n ? ys[b] : nullptr;
    terms.scale[b] = b < terms.n ? scales[b] : 0.f;
  }
  const size_t smem = ((size_t)H + 33) * sizeof(float);
  if (smem > 200 * 1024) MB_FAIL("mb_stream_step: rows of %d values", H);
  cudaStream_t s = (cudaStream_t)stream;
  // four columns a thread where everything lies on 16-byte boundaries
  uintptr_t bits = (uintptr_t)x | (uintptr_t)w | (uintptr_t)out | (uintptr_t)(stream_stride * 4);
  for (int b = 0; b < terms.n; ++b) bits |= (uintptr_t)terms.y[b];
  const bool vec = H % 4 == 0 && (bits & 15) == 0;
  const int per = vec ? 4 : 1;
  const int threads = H >= 2048 * per ? 512 : (H >= 512 * per ? 256 : 128);
#define GOV(TW_, TO_, V_)                                                                     \
  {                                                                                           \
    static size_t configured = 48 * 1024;                                                     \
    if (smem > configured) {                                                                  \
      cudaFuncSetAttribute(stream_step_kernel<TW_, TO_, V_>,                                  \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);          \
      configured = 200 * 1024;                                                                \
    }                                                                                         \
    mb_launch(stream_step_kernel<TW_, TO_, V_>, dim3(R), dim3(threads), smem, s, x,           \
              (size_t)stream_stride, S, mix, outc, terms, in, (const TW_*)w, eps, (TO_*)out,  \
              rows, H);                                                                       \
  }
#define GO(TW_, TO_) { if (vec) GOV(TW_, TO_, 4) else GOV(TW_, TO_, 1) }
  if (w_dtype == MB_F32 && out_dtype == MB_F32) GO(float, float)
  else if (w_dtype == MB_F32) GO(float, __nv_bfloat16)
  else if (out_dtype == MB_F32) GO(__nv_bfloat16, float)
  else GO(__nv_bfloat16, __nv_bfloat16)
#undef GO
#undef GOV
  MB_CHECK_LAUNCH("mb_stream_step");
}

// x (+)= sum_b scale_b y_b over [T, H] float32: the branches of a mixer that runs side by
// side, summed with a factor each, in order. store: x = the sum.
__global__ void add_scaled_kernel(float* __restrict__ x, StTerms terms, size_t total, int store) {
  mb_grid_wait();
  mb_grid_launch_next();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    float y = 0.f;
    for (int b = 0; b < terms.n; ++b)
      y = b == 0 ? terms.scale[0] * terms.y[0][i] : fmaf(terms.scale[b], terms.y[b][i], y);
    x[i] = store ? y : x[i] + y;
  }
}

MB_EXPORT int mb_add_scaled(float* x, const float* const* ys, const float* scales, int n_terms,
                            long long total, int store, void* stream) {
  if (total <= 0) return 0;
  if (n_terms < 1 || n_terms > ST_MAX_TERMS) MB_FAIL("mb_add_scaled: %d terms", n_terms);
  StTerms terms;
  terms.n = n_terms;
  for (int b = 0; b < ST_MAX_TERMS; ++b) {
    terms.y[b] = b < n_terms ? ys[b] : nullptr;
    terms.scale[b] = b < n_terms ? scales[b] : 0.f;
  }
  const long long want = (total + 255) / 256;
  mb_launch(add_scaled_kernel, dim3((unsigned)(want < 148 * 8 ? want : 148 * 8)), dim3(256), 0,
            (cudaStream_t)stream, x, terms, (size_t)total, store);
  MB_CHECK_LAUNCH("mb_add_scaled");
}
