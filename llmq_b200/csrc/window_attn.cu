// window_attn.cu — rotary grouped-query attention over a sliding window.  The paged cache holds, per token, the
// turned keys of every key/value head followed by their values ([kv_heads*dim | kv_heads*vdim], model dtype).
// Rotation pairs dimension i with i + rot_dims/2 over the first rot_dims dimensions of a head (angles and their
// sine / cosine in fp64 from position * freq[i]); the score scale and a per-head temperature are folded into the
// fp32 query; ordinary softmax over the keys max(0, p - window + 1) .. p; one sigmoid gate number per head.
// A scalar kernel (fp32 model, any head size) and tensor-core kernels for bf16 caches.  Scores, softmax state
// and accumulators are fp32 in all.
#include <stdlib.h>

#include <algorithm>

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
// step 1 (CTA per token): sine / cosine of the token's angles once in shared memory, then every query head
// (turned, times scale * temp[h], fp32) and every key head (turned, into the cache row); values are copied.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) window_attn_prep_kernel(const T* __restrict__ proj, int ldp, int heads,
                                                               int kv_heads, int dim, int vdim, int rot_dims,
                                                               const double* __restrict__ freq,
                                                               const int32_t* __restrict__ positions,
                                                               const int32_t* __restrict__ slot_mapping,
                                                               const float* __restrict__ temp, float scale,
                                                               float* __restrict__ qs, T* __restrict__ cache) {
  extern __shared__ float cs[];  // [rot_dims/2] cos | [rot_dims/2] sin
  const int t = blockIdx.x, half = rot_dims / 2;
  const double p = (double)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sn, c;
    sincos(p * freq[i], &sn, &c);
    cs[i] = (float)c;
    cs[half + i] = (float)sn;
  }
  __syncthreads();
  const T* pr = proj + (long long)t * ldp;
  auto turned = [&](const T* v, int d) -> float {
    if (d >= rot_dims) return ldf(v + d);
    const int i = d < half ? d : d - half;
    const float a = ldf(v + i), b = ldf(v + i + half);
    return d < half ? a * cs[i] - b * cs[half + i] : b * cs[i] + a * cs[half + i];
  };
  for (int e = threadIdx.x; e < heads * dim; e += blockDim.x) {
    const int h = e / dim, d = e % dim;
    qs[(long long)t * heads * dim + e] = turned(pr + (long long)h * dim, d) * (scale * (temp ? temp[h] : 1.f));
  }
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const int GD = kv_heads * dim, GV = kv_heads * vdim;
  const T* k = pr + (long long)heads * dim;
  T* row = cache + (long long)slot * (GD + GV);
  for (int e = threadIdx.x; e < GD; e += blockDim.x) stf(row + e, turned(k + (long long)(e / dim) * dim, e % dim));
  for (int e = threadIdx.x; e < GV; e += blockDim.x) row[GD + e] = k[GD + e];
}

// ------------------------------------------------------------------------------------------------
// step 2, scalar form: one CTA per (token, key/value head, group of 8 query heads that share it).  Tiles of 32
// cached keys and values are staged in shared memory once and used by up to 8 query heads (warp = head; lane =
// key for the scores, lane = output dims for the weighted sum).  Tiles start at the window's first key, so a
// token's result does not depend on what else the step holds.
// ------------------------------------------------------------------------------------------------
template <typename T, int ACC>
__global__ void __launch_bounds__(256) window_attn_kernel(const float* __restrict__ qs, const T* __restrict__ cache,
                                                          const int32_t* __restrict__ block_table, int bt_stride,
                                                          const int32_t* __restrict__ row_seq,
                                                          const int32_t* __restrict__ positions, int heads, int kv_heads,
                                                          int dim, int vdim, int block_size, int window,
                                                          const T* __restrict__ gate, int ld_gate, T* __restrict__ out) {
  extern __shared__ float sm[];
  const int KS = dim + 1, VS = vdim + 1;
  float* qsm = sm;              // [8][dim]
  float* ksm = sm + 8 * dim;    // [32][dim+1]
  float* vsm = ksm + 32 * KS;   // [32][vdim+1]
  const int t = blockIdx.x, g = blockIdx.y, rep = heads / kv_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hg = blockIdx.z * 8 + warp;  // head within the group
  const bool live = hg < rep;
  const int h = g * rep + hg;
  const int p = positions[t];
  const int32_t* bt = block_table + (long long)row_seq[t] * bt_stride;
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int GD = kv_heads * dim, RS = GD + kv_heads * vdim;
  for (int e = threadIdx.x; e < 8 * dim; e += blockDim.x) {
    const int hh = blockIdx.z * 8 + e / dim;
    qsm[e] = hh < rep ? qs[((long long)t * heads + g * rep + hh) * dim + e % dim] : 0.f;
  }
  float m = -INFINITY, l = 0.f;
  float acc[ACC];
#pragma unroll
  for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
  const float* qh = qsm + warp * dim;
  for (int j0 = lo; j0 <= p; j0 += 32) {
    const int n = min(32, p + 1 - j0);
    __syncthreads();
    for (int e = threadIdx.x; e < n * (dim + vdim); e += blockDim.x) {
      const int j = e / (dim + vdim), d = e % (dim + vdim), pos = j0 + j;
      const long long row = (long long)bt[pos / block_size] * block_size + pos % block_size;
      if (d < dim) ksm[j * KS + d] = ldf(cache + row * RS + (long long)g * dim + d);
      else vsm[j * VS + d - dim] = ldf(cache + row * RS + GD + (long long)g * vdim + d - dim);
    }
    __syncthreads();
    if (!live) continue;
    float s = -INFINITY;
    if (lane < n) {
      const float* kr = ksm + lane * KS;
      float dot = 0.f;
      for (int d = 0; d < dim; ++d) dot = fmaf(qh[d], kr[d], dot);
      s = dot;
    }
    const float m_new = fmaxf(m, warp_max(s));  // the tile holds at least the key j0 <= p: finite
    const float corr = expf(m - m_new);
    const float pl = lane < n ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pl);
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] *= corr;
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pl, j);
      const float* vr = vsm + j * VS;
#pragma unroll
      for (int i = 0; i < ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < vdim) acc[i] = fmaf(pj, vr[d], acc[i]);
      }
    }
    m = m_new;
  }
  if (!live) return;
  const float gv = gate ? sigmoidf_(ldf(gate + (long long)t * ld_gate + h)) : 1.f;
  const float inv = gv / l;
  T* o = out + ((long long)t * heads + h) * vdim;
#pragma unroll
  for (int i = 0; i < ACC; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) stf(o + d, acc[i] * inv);
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_window_attn_prep(const void* proj, int ldp, int heads, int kv_heads, int dim, int vdim, int rot_dims,
                           const double* freq, const int32_t* positions, const int32_t* slot_mapping, const float* temp,
                           float scale, float* qs, void* cache, int T_, int dtype, void* stream) {
  B200Q_CHECK_ARG(proj && positions && slot_mapping && qs && cache && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 &&
                      ldp >= heads * dim + kv_heads * (dim + vdim) && rot_dims >= 0 && rot_dims % 2 == 0 &&
                      rot_dims <= dim && (rot_dims == 0 || freq) && T_ >= 0 && is_dtype(dtype),
                  "window_attn_prep: bad argument (heads=%d kv_heads=%d dim=%d vdim=%d rot_dims=%d even, <= dim)", heads,
                  kv_heads, dim, vdim, rot_dims);
  if (T_ == 0) return B200Q_OK;
  DISPATCH_T(dtype, (window_attn_prep_kernel<T><<<T_, 128, (size_t)std::max(rot_dims, 1) * sizeof(float),
                                                  as_stream(stream)>>>((const T*)proj, ldp, heads, kv_heads, dim, vdim,
                                                                       rot_dims, freq, positions, slot_mapping, temp, scale,
                                                                       qs, (T*)cache)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_window_attn(const float* qs, const void* cache, const int32_t* block_table, int bt_stride, const int32_t* row_seq,
                      const int32_t* positions, const int32_t* seq_desc, int n_seqs, int T_, int heads, int kv_heads,
                      int dim, int vdim, int block_size, int window, const void* gate, int ld_gate, void* out, int dtype,
                      void* stream) {
  B200Q_CHECK_ARG(qs && cache && block_table && row_seq && positions && out && heads > 0 && kv_heads > 0 &&
                      heads % kv_heads == 0 && dim > 0 && dim <= 512 && vdim > 0 && vdim <= 512 && block_size > 0 &&
                      window >= 0 && T_ >= 0 && is_dtype(dtype) && (!gate || ld_gate >= heads),
                  "window_attn: bad argument (heads=%d kv_heads=%d dim=%d vdim=%d, both <= 512)", heads, kv_heads, dim,
                  vdim);
  if (T_ == 0) return B200Q_OK;
  cudaStream_t st = as_stream(stream);
  const int rep = heads / kv_heads;
  dim3 grid(T_, kv_heads, (rep + 7) / 8);
  B200Q_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "window_attn: too many heads");
  const size_t smem = (size_t)(8 * dim + 32 * (dim + 1) + 32 * (vdim + 1)) * sizeof(float);
#define SCALAR(ACC)                                                                                                       \
  do {                                                                                                                    \
    DISPATCH_T(dtype, {                                                                                                   \
      auto kern = window_attn_kernel<T, ACC>;                                                                             \
      if (smem > 48 * 1024) B200Q_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      kern<<<grid, 256, smem, st>>>(qs, (const T*)cache, block_table, bt_stride, row_seq, positions, heads, kv_heads, dim, \
                                    vdim, block_size, window, (const T*)gate, ld_gate, (T*)out);                          \
    });                                                                                                                   \
  } while (0)
  if (vdim <= 64) SCALAR(2);
  else if (vdim <= 128) SCALAR(4);
  else if (vdim <= 256) SCALAR(8);
  else SCALAR(16);
#undef SCALAR
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // extern "C"
