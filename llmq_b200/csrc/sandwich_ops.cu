// sandwich_ops.cu — elementwise kernels of the sandwich layer form (a norm on both sides of every sublayer, a
// residual multiplier, a per-layer token input) and the rotation-frequency table shared by the attention mixers.
//
//   row_norm:        y = norm(x[rows])                       dynamic tanh, RMS, or a plain cast
//   sandwich_add:    x += mult * post(y + bias);  out = next(x)     one pass over the row, x stays fp32
//   gelu_glu:        y = gelu_tanh(g) * u
//   token_side_gate: out = gelu_tanh(g) * table[token, col0 ..]
//
// Dynamic tanh is tanh(alpha v) * w + b with the weights as one fp32 row [w | b | alpha]: it needs no statistics of
// the row, so the sum that closes a sublayer and the norm that opens the next one are a single pass.  All arithmetic
// is fp32; only y, out and the table are in the model dtype.
#include <math.h>

#include <vector>

#include "layered_common.cuh"

namespace b200q {

__device__ __forceinline__ float gelu_tanhf_(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T> __device__ __forceinline__ void ld4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void ld4<float>(const float* p, float (&v)[4]) {
  const float4 f = *reinterpret_cast<const float4*>(p);
  v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
template <> __device__ __forceinline__ void ld4<bf16>(const bf16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  v[0] = bf16_lo(u.x); v[1] = bf16_hi(u.x); v[2] = bf16_lo(u.y); v[3] = bf16_hi(u.y);
}
template <typename T> __device__ __forceinline__ void st4(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void st4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void st4<bf16>(bf16* p, const float (&v)[4]) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
}

// one norm applied to V consecutive values of a row that start at column c
template <int V>
__device__ __forceinline__ void apply_norm(int kind, const float* __restrict__ w, int W, int c, float inv,
                                           const float (&in)[4], float (&out)[4]) {
  if (kind == B200Q_NORM_DYT) {
    const float alpha = w[2 * W];
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = tanhf(alpha * in[i]) * w[c + i] + w[W + c + i];
  } else if (kind == B200Q_NORM_RMS) {
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = in[i] * inv * w[c + i];
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = in[i];
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256) row_norm_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                                       int kind, const float* __restrict__ w, T* __restrict__ y, int W,
                                                       float eps) {
  __shared__ float red[32];
  const long long src = rows ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + src * W;
  T* yr = y + (long long)blockIdx.x * W;
  float inv = 0.f;
  if (kind == B200Q_NORM_RMS) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
    inv = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
  }
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float a[4], o[4];
    if (V == 4) {
      ld4(xr + c, a);
      apply_norm<V>(kind, w, W, c, inv, a, o);
      st4(yr + c, o);
    } else {
      a[0] = xr[c];
      apply_norm<V>(kind, w, W, c, inv, a, o);
      stf(yr + c, o[0]);
    }
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256) sandwich_add_kernel(float* __restrict__ x, const T* __restrict__ y,
                                                           const float* __restrict__ bias, int post_kind,
                                                           const float* __restrict__ post_w, float mult, int next_kind,
                                                           const float* __restrict__ next_w, T* __restrict__ out, int W,
                                                           float eps) {
  __shared__ float red[32];
  float* xr = x + (long long)blockIdx.x * W;
  const T* yr = y + (long long)blockIdx.x * W;
  T* outr = out + (long long)blockIdx.x * W;
  float inv = 0.f;
  if (post_kind == B200Q_NORM_RMS) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float v = ldf(yr + c) + (bias ? bias[c] : 0.f);
      ss = fmaf(v, v, ss);
    }
    inv = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
  }
  float ss2 = 0.f;
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float a[4], n[4], xv[4], o[4];
    if (V == 4) {
      ld4(yr + c, a);
      ld4(xr + c, xv);
    } else {
      a[0] = ldf(yr + c);
      xv[0] = xr[c];
    }
    if (bias) {
#pragma unroll
      for (int i = 0; i < V; ++i) a[i] += bias[c + i];
    }
    apply_norm<V>(post_kind, post_w, W, c, inv, a, n);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      xv[i] = fmaf(mult, n[i], xv[i]);
      ss2 = fmaf(xv[i], xv[i], ss2);
    }
    if (V == 4) st4(xr + c, xv);
    else xr[c] = xv[0];
    if (next_kind == B200Q_NORM_DYT || next_kind == B200Q_NORM_CAST) {
      apply_norm<V>(next_kind, next_w, W, c, 0.f, xv, o);
      if (V == 4) st4(outr + c, o);
      else stf(outr + c, o[0]);
    }
  }
  if (next_kind == B200Q_NORM_RMS) {  // the row's statistics exist only now: a second pass over the L1-hot row
    const float inv2 = 1.f / sqrtf(block_sum(ss2, red) / (float)W + eps);
    __syncthreads();
    for (int c = threadIdx.x; c < W; c += blockDim.x) stf(outr + c, xr[c] * inv2 * next_w[c]);
  }
}

// where column c's gate and up values lie in a [2F] row: block 0 = [g (F) | u (F)]; block b > 0 = gate and up
// interleaved in blocks of b columns ([g b | u b | g b | u b ...])
__device__ __forceinline__ void glu_columns(int c, int F, int block, int& g_at, int& u_at) {
  if (block > 0) {
    g_at = (c / block) * 2 * block + c % block;
    u_at = g_at + block;
  } else {
    g_at = c;
    u_at = F + c;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gelu_glu_kernel(const T* __restrict__ gu, T* __restrict__ y, long long rows,
                                                       int F, int block) {
  const long long total = rows * F;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const long long r = e / F;
    int g_at, u_at;
    glu_columns((int)(e % F), F, block, g_at, u_at);
    stf(y + e, gelu_tanhf_(ldf(gu + r * 2 * F + g_at)) * ldf(gu + r * 2 * F + u_at));
  }
}
__global__ void __launch_bounds__(256) gelu_glu_v8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ y,
                                                          long long rows, int F, int block) {
  const int per = F / 8;
  const long long total = rows * per;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const long long r = e / per;
    const int c = (int)(e % per) * 8;
    int g_at, u_at;
    glu_columns(c, F, block, g_at, u_at);  // block is a multiple of 8: the eight columns stay together
    const uint4 g = ld_v4(gu + r * 2 * F + g_at), u = ld_v4(gu + r * 2 * F + u_at);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      o[i] = pack_bf16x2(gelu_tanhf_(bf16_lo(gw[i])) * bf16_lo(uw[i]), gelu_tanhf_(bf16_hi(gw[i])) * bf16_hi(uw[i]));
    st_v4(y + r * F + c, make_uint4(o[0], o[1], o[2], o[3]));
  }
}

__global__ void __launch_bounds__(256) scale_f32_kernel(float* __restrict__ v, long long n, float a) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x)
    v[e] *= a;
}

template <typename T>
__global__ void __launch_bounds__(256) token_side_gate_kernel(const T* __restrict__ g, int ldg,
                                                              const int32_t* __restrict__ ids,
                                                              const int32_t* __restrict__ prev_out,
                                                              const T* __restrict__ table, int ld_table, int col0,
                                                              T* __restrict__ out, int Tn, int D) {
  const long long total = (long long)Tn * D;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(e / D), j = (int)(e % D);
    int id = __ldg(ids + t);
    if (id < 0) id = prev_out[-1 - id];
    stf(out + e, gelu_tanhf_(ldf(g + (long long)t * ldg + j)) * ldf(table + (long long)id * ld_table + col0 + j));
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_rot_frequencies(int rot_dims, double base, double factor, double original, double fast, double slow,
                          double* freq_out, float* mag_out) {
  B200Q_CHECK_ARG(rot_dims >= 0 && rot_dims % 2 == 0 && (rot_dims == 0 || (base > 0.0 && freq_out)) && factor >= 0.0 &&
                      original >= 0.0 && (original == 0.0 || (factor > 0.0 && fast > 0.0 && slow > 0.0 && base != 1.0)),
                  "rot_frequencies: bad argument (dims=%d base=%g factor=%g original=%g fast=%g slow=%g)", rot_dims, base,
                  factor, original, fast, slow);
  const int half = rot_dims / 2;
  double mag = 1.0;
  double lo = 0.0, hi = 0.0;
  if (original > 0.0) {
    auto at = [&](double turns) { return rot_dims * log(original / (2.0 * M_PI * turns)) / (2.0 * log(base)); };
    lo = fmax(floor(at(fast)), 0.0);
    hi = fmin(ceil(at(slow)), (double)(rot_dims - 1));
    mag = 0.1 * log(factor) + 1.0;
  }
  for (int i = 0; i < half; ++i) {
    const double f = pow(base, -2.0 * i / (double)rot_dims);
    if (original > 0.0) {
      const double r = fmin(fmax(((double)i - lo) / fmax(hi - lo, 0.001), 0.0), 1.0);
      freq_out[i] = f / factor * r + f * (1.0 - r);
    } else {
      freq_out[i] = factor > 0.0 ? f / factor : f;
    }
  }
  if (mag_out) *mag_out = (float)mag;
  return B200Q_OK;
}

static bool norm_kind_ok(int k, bool as_post) {
  return k == B200Q_NORM_DYT || k == B200Q_NORM_RMS || (!as_post && (k == B200Q_NORM_CAST || k == B200Q_NORM_NONE));
}

int b200q_row_norm(const float* x, const int32_t* rows, int kind, const float* w, void* y, int n, int W, float eps,
                   int dtype, void* stream) {
  B200Q_CHECK_ARG(x && y && n >= 0 && W > 0 && is_dtype(dtype) && norm_kind_ok(kind, false) && kind != B200Q_NORM_NONE &&
                      (kind == B200Q_NORM_CAST || w),
                  "row_norm: bad argument (kind=%d)", kind);
  if (n == 0) return B200Q_OK;
  const bool v4 = W % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (v4) DISPATCH_T(dtype, (row_norm_kernel<T, 4><<<n, 256, 0, as_stream(stream)>>>(x, rows, kind, w, (T*)y, W, eps)));
  else DISPATCH_T(dtype, (row_norm_kernel<T, 1><<<n, 256, 0, as_stream(stream)>>>(x, rows, kind, w, (T*)y, W, eps)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_sandwich_add(float* x, const void* y, const float* bias, int post_kind, const float* post_w, float mult,
                       int next_kind, const float* next_w, void* out, int T_, int W, float eps, int dtype, void* stream) {
  B200Q_CHECK_ARG(x && y && post_w && T_ >= 0 && W > 0 && is_dtype(dtype) && norm_kind_ok(post_kind, true) &&
                      norm_kind_ok(next_kind, false) && (next_kind == B200Q_NORM_NONE || out) &&
                      (next_kind == B200Q_NORM_NONE || next_kind == B200Q_NORM_CAST || next_w),
                  "sandwich_add: bad argument (post=%d next=%d)", post_kind, next_kind);
  if (T_ == 0) return B200Q_OK;
  const bool v4 = W % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                                  reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (v4)
    DISPATCH_T(dtype, (sandwich_add_kernel<T, 4><<<T_, 256, 0, as_stream(stream)>>>(
                          x, (const T*)y, bias, post_kind, post_w, mult, next_kind, next_w, (T*)out, W, eps)));
  else
    DISPATCH_T(dtype, (sandwich_add_kernel<T, 1><<<T_, 256, 0, as_stream(stream)>>>(
                          x, (const T*)y, bias, post_kind, post_w, mult, next_kind, next_w, (T*)out, W, eps)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_gelu_glu(const void* gate_up, void* y, int64_t rows, int F, int dtype, void* stream) {
  return b200q_gelu_glu_ex(gate_up, y, rows, F, 0, dtype, stream);
}

int b200q_gelu_glu_ex(const void* gate_up, void* y, int64_t rows, int F, int block, int dtype, void* stream) {
  B200Q_CHECK_ARG(gate_up && y && rows >= 0 && F > 0 && is_dtype(dtype) && block >= 0 && (block == 0 || F % block == 0),
                  "gelu_glu: bad argument (F=%d, blocks of %d)", F, block);
  if (rows == 0) return B200Q_OK;
  if (dtype == B200Q_DTYPE_BF16 && F % 8 == 0 && block % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
    gelu_glu_v8_kernel<<<grid_for(rows * (F / 8)), 256, 0, as_stream(stream)>>>((const bf16*)gate_up, (bf16*)y, rows, F,
                                                                               block);
    B200Q_LAUNCH_CHECK();
    return B200Q_OK;
  }
  DISPATCH_T(dtype, (gelu_glu_kernel<T><<<grid_for(rows * F), 256, 0, as_stream(stream)>>>((const T*)gate_up, (T*)y,
                                                                                         rows, F, block)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_scale_f32(float* v, int64_t n, float a, void* stream) {
  B200Q_CHECK_ARG(v && n >= 0, "scale_f32: bad argument");
  if (n == 0) return B200Q_OK;
  scale_f32_kernel<<<grid_for(n), 256, 0, as_stream(stream)>>>(v, n, a);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_token_side_gate(const void* g, int ldg, const int32_t* ids, const int32_t* prev_out, const void* table,
                          int ld_table, int col0, void* out, int T_, int D, int dtype, void* stream) {
  B200Q_CHECK_ARG(g && ids && table && out && T_ >= 0 && D > 0 && ldg >= D && col0 >= 0 && ld_table >= col0 + D &&
                      is_dtype(dtype),
                  "token_side_gate: bad argument (D=%d ldg=%d col0=%d ld_table=%d)", D, ldg, col0, ld_table);
  if (T_ == 0) return B200Q_OK;
  DISPATCH_T(dtype, (token_side_gate_kernel<T><<<grid_for((long long)T_ * D), 256, 0, as_stream(stream)>>>(
                        (const T*)g, ldg, ids, prev_out, (const T*)table, ld_table, col0, (T*)out, T_, D)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // extern "C"
