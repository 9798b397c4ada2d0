// prenorm_ops.cu — kernels of the sequential pre-norm layer form: plain RMS norm with a token shift whose
// previous row travels in the sequence's state slot, blends of a row with its predecessor, the squared-ReLU
// unit, routing of a grouped mixture with identity experts, residual sums, re-injection input, logit soft cap.
// Norms, blends, router arithmetic and the residual are fp32 whatever the model's element type is.
#include <stdlib.h>

#include "layered_common.cuh"

namespace b200q {

struct SeqView {
  int row0, n, pos0, slot;
};
__device__ __forceinline__ SeqView seq_view(const int32_t* __restrict__ seq_desc, int s) {
  const int4 v = *reinterpret_cast<const int4*>(seq_desc + 4 * s);
  return {v.x, v.y, v.z, v.w};
}

// ------------------------------------------------------------------------------------------------
// RMS norm (+ token shift).  CTA per output row.  With a shift the CTA also norms the previous row of the
// same portion (the residual is hot in L2; no [T, W] buffer of unshifted rows is kept), or takes the
// sequence's carried row for the first token of a portion.  The sum of squares of a row has one order, so a
// row's result does not depend on which CTA computes it.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_shift_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                                            const float* __restrict__ w, const float* __restrict__ shift,
                                                            const float* __restrict__ state, long long slot_stride,
                                                            const int32_t* __restrict__ seq_desc,
                                                            const int32_t* __restrict__ row_seq, float* __restrict__ carry,
                                                            float* __restrict__ state_w, T* __restrict__ y_t,
                                                            float* __restrict__ y_f32, int W, float eps) {
  __shared__ float red[32];
  const int i = blockIdx.x;
  const int t = rows ? rows[i] : i;
  const float* xr = x + (long long)t * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
  if (!shift) {
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float v = xr[c] * inv * w[c];
      if (y_t) stf(y_t + (long long)i * W + c, v);
      if (y_f32) y_f32[(long long)i * W + c] = v;
    }
    return;
  }
  const int s = row_seq[t];
  const SeqView sq = seq_view(seq_desc, s);
  const bool first = t == sq.row0, last = t == sq.row0 + sq.n - 1;
  const float* pr = nullptr;  // the previous row's source: a residual row, the carried row, or nothing (zeros)
  float pinv = 1.f;
  if (!first) {
    const float* xp = xr - W;
    float ps = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) ps = fmaf(xp[c], xp[c], ps);
    pinv = 1.f / sqrtf(block_sum(ps, red) / (float)W + eps);
    pr = xp;
  } else if (sq.pos0 > 0) {
    pr = state + (long long)sq.slot * slot_stride;
  }
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float n = xr[c] * inv * w[c];
    const float p = pr ? (first ? pr[c] : pr[c] * pinv * w[c]) : 0.f;
    const float v = n + (p - n) * shift[c];
    if (y_t) stf(y_t + (long long)i * W + c, v);
    if (y_f32) y_f32[(long long)i * W + c] = v;
    // a portion of one token is read and written by this CTA alone (each thread its own channels): the row goes
    // straight into the slot; longer portions leave it in `carry` until every reader of the old row has run
    if (last) (first ? state_w + (long long)sq.slot * slot_stride : carry + (long long)s * W)[c] = n;
  }
}

// x <- x + sa * a (+ sb * b), then y = x / rms(x) * w: the sum that closes a mixer and the norm that opens the
// feed-forward in one pass over the row (CTA per row; the row stays in registers between the two)
constexpr int ADDNORM_MAX = 16;  // channels per thread: rows of up to 4096 values stay in registers
template <typename T>
__global__ void __launch_bounds__(256) residual_add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ a, float sa,
                                                                   const T* __restrict__ b, float sb,
                                                                   const float* __restrict__ w, T* __restrict__ y, int W,
                                                                   float eps) {
  __shared__ float red[32];
  const long long base = (long long)blockIdx.x * W;
  const bool keep = W <= ADDNORM_MAX * (int)blockDim.x;
  float v[ADDNORM_MAX];
  float ss = 0.f;
  int q = 0;
  for (int c = threadIdx.x; c < W; c += blockDim.x, ++q) {
    float t = sa * ldf(a + base + c);
    if (b) t = fmaf(sb, ldf(b + base + c), t);
    t += x[base + c];
    x[base + c] = t;
    if (keep) v[q < ADDNORM_MAX ? q : 0] = t;
    ss = fmaf(t, t, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
  q = 0;
  for (int c = threadIdx.x; c < W; c += blockDim.x, ++q)
    stf(y + base + c, (keep ? v[q < ADDNORM_MAX ? q : 0] : x[base + c]) * inv * w[c]);
}

__global__ void __launch_bounds__(256) store_carry_kernel(const float* __restrict__ src, int last_rows,
                                                          float* __restrict__ state, long long slot_stride,
                                                          const int32_t* __restrict__ seq_desc, int W, int skip_single) {
  const SeqView sq = seq_view(seq_desc, blockIdx.x);
  if (sq.n <= 0 || (skip_single && sq.n == 1)) return;  // single tokens were stored by their reader
  const float* r = src + (long long)(last_rows ? sq.row0 + sq.n - 1 : blockIdx.x) * W;
  float* d = state + (long long)sq.slot * slot_stride;
  for (int c = threadIdx.x; c < W; c += blockDim.x) d[c] = r[c];
}

template <typename T>
__global__ void __launch_bounds__(256) shift_blend_kernel(const float* __restrict__ h, const float* __restrict__ mu,
                                                          int n_mix, const float* __restrict__ state,
                                                          long long slot_stride, const int32_t* __restrict__ seq_desc,
                                                          const int32_t* __restrict__ row_seq, float* __restrict__ state_w,
                                                          T* __restrict__ out, int W) {
  const int t = blockIdx.x;
  const SeqView sq = seq_view(seq_desc, row_seq[t]);
  const float* hr = h + (long long)t * W;
  const float* pr = t > sq.row0 ? hr - W : (sq.pos0 > 0 ? state + (long long)sq.slot * slot_stride : nullptr);
  float* keep = (state_w && sq.n == 1) ? state_w + (long long)sq.slot * slot_stride : nullptr;  // see rmsnorm_shift
  T* o = out + (long long)t * n_mix * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = hr[c], d = (pr ? pr[c] : 0.f) - v;
    for (int s = 0; s < n_mix; ++s) stf(o + (long long)s * W + c, fmaf(d, mu[(long long)s * W + c], v));
    if (keep) keep[c] = v;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) relu2_kernel(T* __restrict__ z, long long n) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {
    const float v = fmaxf(ldf(z + e), 0.f);
    stf(z + e, v * v);
  }
}
__global__ void __launch_bounds__(256) relu2_v8_kernel(bf16* __restrict__ z, long long n8) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n8; e += (long long)gridDim.x * blockDim.x) {
    uint4 v = ld_v4(z + e * 8);
    uint32_t* p = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = fmaxf(bf16_lo(p[i]), 0.f), b = fmaxf(bf16_hi(p[i]), 0.f);
      p[i] = pack_bf16x2(a * a, b * b);
    }
    st_v4(z + e * 8, v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) tanh_cast_kernel(const float* __restrict__ in, T* __restrict__ out, long long n) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x)
    stf(out + e, tanhf(in[e]));
}

template <typename T>
__global__ void __launch_bounds__(256) act_to_f32_kernel(const T* __restrict__ in, int ld_in, float* __restrict__ out,
                                                         int ld_out, int C, int act, long long total) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long t = e / C;
    const int c = (int)(e % C);
    const float v = ldf(in + t * ld_in + c);
    out[t * ld_out + c] = act == 1 ? siluf_(v) : v;
  }
}

// bf16 rows, 8 values per thread (16-byte load, two 16-byte stores); C, both strides and both bases aligned
__global__ void __launch_bounds__(256) act_to_f32_v8_kernel(const bf16* __restrict__ in, int ld_in, float* __restrict__ out,
                                                            int ld_out, int C8, int act, long long total8) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total8; e += (long long)gridDim.x * blockDim.x) {
    const long long t = e / C8;
    const int c = (int)(e - t * C8) * 8;
    const uint4 v = ld_v4(in + t * ld_in + c);
    const uint32_t p[4] = {v.x, v.y, v.z, v.w};
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = bf16_lo(p[i]);
      f[2 * i + 1] = bf16_hi(p[i]);
    }
    if (act == 1) {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = siluf_(f[i]);
    }
    float4* o = reinterpret_cast<float4*>(out + t * ld_out + c);
    o[0] = make_float4(f[0], f[1], f[2], f[3]);
    o[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
}

// a decay acts at every later token of its sequence: the fp32 model takes both exponentials through fp64
template <bool EXACT>
__global__ void __launch_bounds__(256) decay_from_logits_kernel(float* __restrict__ w, int ldw,
                                                                const float* __restrict__ w0, int C, long long total) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    float* p = w + (e / C) * ldw + e % C;
    const float z = *p + w0[e % C];
    *p = EXACT ? (float)exp(-exp((double)z)) : expf(-expf(z));
  }
}

// ------------------------------------------------------------------------------------------------
// grouped routing: one warp per token.  Scores are the softmax over ALL experts; the choice adds the
// correction and is masked to the kept groups (a masked expert counts as minus infinity, so negative choice
// scores still beat it).  Ties go to the lowest index, for groups and for experts.
// ------------------------------------------------------------------------------------------------
constexpr int ROUTE_MAX_GROUPS = 256;
__global__ void __launch_bounds__(128) moe_route_grouped_kernel(const float* __restrict__ logits,
                                                                const float* __restrict__ corr, int Tn, int E, int top,
                                                                int n_groups, int keep, int32_t* __restrict__ idx,
                                                                float* __restrict__ wts) {
  __shared__ float gscore[4][ROUTE_MAX_GROUPS];
  const int wi = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + wi;
  if (t >= Tn) return;
  const float* z = logits + (long long)t * E;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) sum += expf(z[e] - mx);
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  auto score = [&](int e) { return expf(z[e] - mx) * inv; };
  const int gs = E / n_groups;
  float* gsc = gscore[wi];
  for (int g = lane; g < n_groups; g += 32) {
    float b = -INFINITY;
    for (int e = g * gs; e < (g + 1) * gs; ++e) b = fmaxf(b, score(e) + corr[e]);
    gsc[g] = b;
  }
  __syncwarp();
  // a group is kept if fewer than `keep` groups rank before it (larger score, or equal score and lower index);
  // every lane decides for its groups first, then the scores are replaced by the flags
  {
    float keepv[ROUTE_MAX_GROUPS / 32];
    int q = 0;
    for (int g = lane; g < n_groups; g += 32, ++q) {
      const float v = gsc[g];
      int before = 0;
      for (int o = 0; o < n_groups; ++o) before += (gsc[o] > v || (gsc[o] == v && o < g)) ? 1 : 0;
      keepv[q] = before < keep ? 1.f : 0.f;
    }
    __syncwarp();
    q = 0;
    for (int g = lane; g < n_groups; g += 32, ++q) gsc[g] = keepv[q];
    __syncwarp();
  }
  float chosen_s = 0.f;
  int chosen_i = -1;
  float prev_v = INFINITY;
  int prev_i = -1;
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY, bs = 0.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      if (gsc[e / gs] == 0.f) continue;
      const float s = score(e), v = s + corr[e];
      const bool below = v < prev_v || (v == prev_v && e > prev_i);
      if (below && (v > bv || (v == bv && e < bi))) {
        bv = v;
        bi = e;
        bs = s;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o), os = __shfl_xor_sync(0xffffffffu, bs, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
        bs = os;
      }
    }
    if (lane == k) {
      chosen_s = bs;
      chosen_i = bi;
    }
    prev_v = bv;
    prev_i = bi;
  }
  const float tot = warp_sum(lane < top ? chosen_s : 0.f);
  if (lane < top) {
    idx[(long long)t * top + lane] = chosen_i;
    wts[(long long)t * top + lane] = chosen_s / (tot + 1e-20f);
  }
}

// grouping of the pairs by expert (one CTA), as for the other mixtures, with the tile table limited to the
// experts that run a product
__global__ void __launch_bounds__(1024) moe_plan_part_kernel(const int32_t* __restrict__ idx, int P, int top, int E,
                                                             int e_gemm, int32_t* __restrict__ group_off,
                                                             int32_t* __restrict__ perm_tok, int32_t* __restrict__ pair_pos,
                                                             int32_t* __restrict__ tile_tab, int32_t* __restrict__ n_tiles) {
  extern __shared__ int32_t si[];  // counts[E] | offs[E+1] | cursor[E]
  int32_t* counts = si;
  int32_t* offs = si + E;
  int32_t* cursor = offs + E + 1;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&counts[idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      offs[e] = run;
      run += counts[e];
    }
    offs[E] = run;
    if (tile_tab) {
      int n = 0;
      for (int e = 0; e < e_gemm; ++e)
        for (int r = offs[e]; r < offs[e + 1]; r += 128) {
          tile_tab[4 * n + 0] = e;
          tile_tab[4 * n + 1] = r;
          tile_tab[4 * n + 2] = offs[e + 1];
          tile_tab[4 * n + 3] = 0;
          ++n;
        }
      *n_tiles = n;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) group_off[e] = offs[e];
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = idx[p];
    const int pos = offs[e] + atomicAdd(&cursor[e], 1);
    perm_tok[pos] = p / top;
    pair_pos[p] = pos;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) residual_add_kernel(float* __restrict__ x, const T* __restrict__ a, float sa,
                                                           const T* __restrict__ b, float sb, long long total) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    float v = sa * ldf(a + e);
    if (b) v = fmaf(sb, ldf(b + e), v);
    x[e] += v;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) residual_add_routed_kernel(float* __restrict__ x, const T* __restrict__ eout,
                                                                  const int32_t* __restrict__ pair_pos,
                                                                  const int32_t* __restrict__ idx,
                                                                  const float* __restrict__ wts, int top, int n_real,
                                                                  const T* __restrict__ h, int Tn, int W) {
  const long long total = (long long)Tn * W;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(e / W), c = (int)(e % W);
    float ff = 0.f;
    for (int k = 0; k < top; ++k) {
      const long long p = (long long)t * top + k;
      const float v = idx[p] < n_real ? ldf(eout + (long long)pair_pos[p] * W + c) : ldf(h + e);
      ff = fmaf(wts[p], v, ff);
    }
    x[e] += ff;
  }
}

// bf16 rows, 8 channels per thread: the token's chosen rows are read with 16-byte loads
__global__ void __launch_bounds__(256) residual_add_routed_v8_kernel(float* __restrict__ x, const bf16* __restrict__ eout,
                                                                     const int32_t* __restrict__ pair_pos,
                                                                     const int32_t* __restrict__ idx,
                                                                     const float* __restrict__ wts, int top, int n_real,
                                                                     const bf16* __restrict__ h, int Tn, int W8) {
  const long long total = (long long)Tn * W8;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(e / W8), c = (int)(e - (long long)t * W8) * 8;
    const long long at = (long long)t * W8 * 8 + c;
    float ff[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top; ++k) {
      const long long p = (long long)t * top + k;
      const uint4 v = idx[p] < n_real ? ld_v4(eout + (long long)pair_pos[p] * W8 * 8 + c) : ld_v4(h + at);
      const uint32_t q[4] = {v.x, v.y, v.z, v.w};
      const float wk = wts[p];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ff[2 * i] = fmaf(wk, bf16_lo(q[i]), ff[2 * i]);
        ff[2 * i + 1] = fmaf(wk, bf16_hi(q[i]), ff[2 * i + 1]);
      }
    }
    float4* xo = reinterpret_cast<float4*>(x + at);
    float4 a = xo[0], b = xo[1];
    a.x += ff[0]; a.y += ff[1]; a.z += ff[2]; a.w += ff[3];
    b.x += ff[4]; b.y += ff[5]; b.z += ff[6]; b.w += ff[7];
    xo[0] = a;
    xo[1] = b;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                          T* __restrict__ out, int Tn, int W) {
  const long long total = (long long)Tn * 2 * W;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long t = e / (2 * W);
    const int c = (int)(e % (2 * W));
    stf(out + e, c < W ? a[t * W + c] : b[t * W + c - W]);
  }
}

__global__ void __launch_bounds__(256) softcap_f32_kernel(float* __restrict__ l, long long n, float cap, float inv_cap) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x)
    l[e] = cap * tanhf(l[e] * inv_cap);
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_rmsnorm_shift(const float* x, const int32_t* rows, const float* w, const float* shift, float* state,
                        long long slot_stride, const int32_t* seq_desc, const int32_t* row_seq, int n_seqs, float* carry,
                        void* y_t, float* y_f32, int n, int W, float eps, int dtype, void* stream) {
  B200Q_CHECK_ARG(x && w && (y_t || y_f32) && n >= 0 && W > 0 && eps > 0.f && is_dtype(dtype),
                  "rmsnorm_shift: bad argument (n=%d W=%d)", n, W);
  B200Q_CHECK_ARG(!shift || (state && seq_desc && row_seq && carry && n_seqs > 0 && !rows),
                  "rmsnorm_shift: a shift needs the state, the per-sequence view and the carry buffer, and no row gather");
  if (n == 0) return B200Q_OK;
  DISPATCH_T(dtype, (rmsnorm_shift_kernel<T><<<n, 256, 0, as_stream(stream)>>>(x, rows, w, shift, state, slot_stride,
                                                                               seq_desc, row_seq, carry, state, (T*)y_t,
                                                                               y_f32, W, eps)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_store_carry(const float* src, int last_rows, float* state, long long slot_stride, const int32_t* seq_desc,
                      int n_seqs, int W, int skip_single, void* stream) {
  B200Q_CHECK_ARG(src && state && seq_desc && n_seqs >= 0 && W > 0, "store_carry: bad argument");
  if (n_seqs == 0) return B200Q_OK;
  store_carry_kernel<<<n_seqs, 256, 0, as_stream(stream)>>>(src, last_rows, state, slot_stride, seq_desc, W, skip_single);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_shift_blend(const float* h, const float* mu, int n_mix, float* state, long long slot_stride,
                      const int32_t* seq_desc, const int32_t* row_seq, int store_single, void* out, int T_, int W, int dtype,
                      void* stream) {
  B200Q_CHECK_ARG(h && mu && n_mix > 0 && state && seq_desc && row_seq && out && T_ >= 0 && W > 0 && is_dtype(dtype),
                  "shift_blend: bad argument");
  if (T_ == 0) return B200Q_OK;
  DISPATCH_T(dtype, (shift_blend_kernel<T><<<T_, 256, 0, as_stream(stream)>>>(h, mu, n_mix, state, slot_stride, seq_desc,
                                                                              row_seq, store_single ? state : nullptr,
                                                                              (T*)out, W)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_relu2(void* z, int64_t n, int dtype, void* stream) {
  B200Q_CHECK_ARG(z && n >= 0 && is_dtype(dtype), "relu2: bad argument");
  if (n == 0) return B200Q_OK;
  if (dtype == B200Q_DTYPE_BF16 && n % 8 == 0 && (reinterpret_cast<uintptr_t>(z) & 15) == 0)
    relu2_v8_kernel<<<grid_for(n / 8), 256, 0, as_stream(stream)>>>((bf16*)z, n / 8);
  else
    DISPATCH_T(dtype, (relu2_kernel<T><<<grid_for(n), 256, 0, as_stream(stream)>>>((T*)z, n)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_tanh_cast(const float* in, void* out, int64_t n, int dtype, void* stream) {
  B200Q_CHECK_ARG(in && out && n >= 0 && is_dtype(dtype), "tanh_cast: bad argument");
  if (n == 0) return B200Q_OK;
  DISPATCH_T(dtype, (tanh_cast_kernel<T><<<grid_for(n), 256, 0, as_stream(stream)>>>(in, (T*)out, n)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_act_to_f32(const void* in, int ld_in, float* out, int ld_out, int C, int act, int T_, int dtype, void* stream) {
  B200Q_CHECK_ARG(in && out && C > 0 && ld_in >= C && ld_out >= C && (act == 0 || act == 1) && T_ >= 0 && is_dtype(dtype),
                  "act_to_f32: bad argument");
  if (T_ == 0) return B200Q_OK;
  const long long total = (long long)T_ * C;
  if (dtype == B200Q_DTYPE_BF16 && C % 8 == 0 && ld_in % 8 == 0 && ld_out % 4 == 0 &&
      ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0)
    act_to_f32_v8_kernel<<<grid_for(total / 8), 256, 0, as_stream(stream)>>>((const bf16*)in, ld_in, out, ld_out, C / 8, act,
                                                                             total / 8);
  else
    DISPATCH_T(dtype, (act_to_f32_kernel<T><<<grid_for(total), 256, 0, as_stream(stream)>>>((const T*)in, ld_in, out,
                                                                                            ld_out, C, act, total)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_decay_from_logits(float* w, int ldw, const float* w0, int C, int T_, int dtype, void* stream) {
  B200Q_CHECK_ARG(w && w0 && C > 0 && ldw >= C && T_ >= 0 && is_dtype(dtype), "decay_from_logits: bad argument");
  if (T_ == 0) return B200Q_OK;
  const long long total = (long long)T_ * C;
  if (dtype == B200Q_DTYPE_F32)
    decay_from_logits_kernel<true><<<grid_for(total), 256, 0, as_stream(stream)>>>(w, ldw, w0, C, total);
  else
    decay_from_logits_kernel<false><<<grid_for(total), 256, 0, as_stream(stream)>>>(w, ldw, w0, C, total);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_moe_route_grouped(const float* logits, const float* correction, int T_, int E, int e_gemm, int top,
                            int n_groups, int keep, int32_t* idx, float* wts, int32_t* group_off, int32_t* perm_tok,
                            int32_t* pair_pos, int32_t* tile_tab, int32_t* n_tiles, void* stream) {
  B200Q_CHECK_ARG(!tile_tab == !n_tiles, "moe_route_grouped: tile_tab and n_tiles go together");
  B200Q_CHECK_ARG(logits && correction && idx && wts && group_off && perm_tok && pair_pos && T_ >= 0 && E > 0 &&
                      E <= 4096 && e_gemm >= 0 && e_gemm <= E && top > 0 && top <= 32 && n_groups > 0 &&
                      n_groups <= ROUTE_MAX_GROUPS && E % n_groups == 0 && keep > 0 && keep <= n_groups &&
                      top <= keep * (E / n_groups),
                  "moe_route_grouped: bad argument (E=%d top=%d groups=%d keep=%d; groups divide E, at most %d groups, "
                  "top fits the kept groups)", E, top, n_groups, keep, ROUTE_MAX_GROUPS);
  if (T_ == 0) return B200Q_OK;
  moe_route_grouped_kernel<<<(T_ + 3) / 4, 128, 0, as_stream(stream)>>>(logits, correction, T_, E, top, n_groups, keep, idx,
                                                                       wts);
  B200Q_LAUNCH_CHECK();
  moe_plan_part_kernel<<<1, 1024, (size_t)(3 * E + 1) * sizeof(int32_t), as_stream(stream)>>>(
      idx, T_ * top, top, E, e_gemm, group_off, perm_tok, pair_pos, tile_tab, n_tiles);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_residual_add(float* x, const void* a, float a_scale, const void* b, float b_scale, int T_, int W, int dtype,
                       void* stream) {
  B200Q_CHECK_ARG(x && a && T_ >= 0 && W > 0 && is_dtype(dtype), "residual_add: bad argument");
  if (T_ == 0) return B200Q_OK;
  const long long total = (long long)T_ * W;
  DISPATCH_T(dtype, (residual_add_kernel<T><<<grid_for(total), 256, 0, as_stream(stream)>>>(x, (const T*)a, a_scale,
                                                                                            (const T*)b, b_scale, total)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_residual_add_rmsnorm(float* x, const void* a, float a_scale, const void* b, float b_scale, const float* w,
                               void* y, int T_, int W, float eps, int dtype, void* stream) {
  B200Q_CHECK_ARG(x && a && w && y && T_ >= 0 && W > 0 && eps > 0.f && is_dtype(dtype), "residual_add_rmsnorm: bad argument");
  if (T_ == 0) return B200Q_OK;
  DISPATCH_T(dtype, (residual_add_rmsnorm_kernel<T><<<T_, 256, 0, as_stream(stream)>>>(x, (const T*)a, a_scale, (const T*)b,
                                                                                       b_scale, w, (T*)y, W, eps)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_residual_add_routed(float* x, const void* expert_out, const int32_t* pair_pos, const int32_t* idx,
                              const float* wts, int top, int n_real, const void* h, int T_, int W, int dtype,
                              void* stream) {
  B200Q_CHECK_ARG(x && expert_out && pair_pos && idx && wts && h && top > 0 && n_real >= 0 && T_ >= 0 && W > 0 &&
                      is_dtype(dtype),
                  "residual_add_routed: bad argument");
  if (T_ == 0) return B200Q_OK;
  if (dtype == B200Q_DTYPE_BF16 && W % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(expert_out) | reinterpret_cast<uintptr_t>(h)) & 15) == 0)
    residual_add_routed_v8_kernel<<<grid_for((long long)T_ * W / 8), 256, 0, as_stream(stream)>>>(
        x, (const bf16*)expert_out, pair_pos, idx, wts, top, n_real, (const bf16*)h, T_, W / 8);
  else
    DISPATCH_T(dtype, (residual_add_routed_kernel<T><<<grid_for((long long)T_ * W), 256, 0, as_stream(stream)>>>(
                          x, (const T*)expert_out, pair_pos, idx, wts, top, n_real, (const T*)h, T_, W)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_concat_cast(const float* a, const float* b, void* out, int T_, int W, int dtype, void* stream) {
  B200Q_CHECK_ARG(a && b && out && T_ >= 0 && W > 0 && is_dtype(dtype), "concat_cast: bad argument");
  if (T_ == 0) return B200Q_OK;
  DISPATCH_T(dtype, (concat_cast_kernel<T><<<grid_for((long long)T_ * 2 * W), 256, 0, as_stream(stream)>>>(a, b, (T*)out,
                                                                                                           T_, W)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_softcap_f32(float* logits, int64_t n, float cap, void* stream) {
  B200Q_CHECK_ARG(logits && n >= 0 && cap > 0.f, "softcap_f32: bad argument");
  if (n == 0) return B200Q_OK;
  softcap_f32_kernel<<<grid_for(n), 256, 0, as_stream(stream)>>>(logits, n, cap, 1.f / cap);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // extern "C"
