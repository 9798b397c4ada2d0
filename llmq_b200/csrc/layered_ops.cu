// layered_ops.cu — kernels of the layered architectures (parallel pre-norm form): fp32 residual stream,
// zero-centred RMS norms, a shape-agnostic linear layer (plain / per-head batched / grouped by expert),
// latent attention over a paged latent cache with a sliding window, the generalized delta-rule
// recurrence over fp32 state slots, PolyNorm, clamped gated experts with top-k routing.
//
// Every kernel is a template over the element type of matrices, activations and cache (bf16 or
// fp32); what has to be exact — residual sum, norms, scores and softmax, router, recurrent state,
// decays and gates of the recurrence, angles — is fp32 (angles fp64) in both instantiations.
// Nothing here depends on which other rows share the batch: every reduction runs in a fixed order
// per row, so a token's result is the same alone, in a chunk or in a mixed batch.
#include <stdlib.h>

#include "layered_common.cuh"

namespace b200q {

// ------------------------------------------------------------------------------------------------
// embedding into the fp32 residual: x[t,:] = table[id,:] * scale (ids < 0: see resolve in elementwise.cu)
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) embed_f32_kernel(const int32_t* __restrict__ ids,
                                                        const int32_t* __restrict__ prev_out,
                                                        const T* __restrict__ table, float* __restrict__ out,
                                                        int Tn, int W, float scale) {
  const long long total = (long long)Tn * W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / W), c = (int)(i % W);
    int id = __ldg(ids + t);
    if (id < 0) id = prev_out[-1 - id];
    out[i] = ldf(table + (long long)id * W + c) * scale;
  }
}

// ------------------------------------------------------------------------------------------------
// zero-centred RMS norm of fp32 rows with up to two weights at once (the two branches of a parallel
// layer read the same x):  y_k = x / sqrt(mean(x^2) + eps) * (1 + w_k).  rows != NULL: gather.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) centered_norm_kernel(const float* __restrict__ x,
                                                            const int32_t* __restrict__ rows,
                                                            const float* __restrict__ w1,
                                                            const float* __restrict__ w2, T* __restrict__ y1,
                                                            T* __restrict__ y2, int W, float eps) {
  __shared__ float red[32];
  const int r = blockIdx.x;
  const float* xr = x + (long long)(rows ? rows[r] : r) * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) ss += xr[c] * xr[c];
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = xr[c] * inv;
    stf(y1 + (long long)r * W + c, v * (1.f + w1[c]));
    if (y2) stf(y2 + (long long)r * W + c, v * (1.f + w2[c]));
  }
}

// ------------------------------------------------------------------------------------------------
// linear layer for ANY shape: C[m,n] = sum_k A[m,k] W[n,k] (+ bias[n]), fp32 FMA accumulation in
// ascending k (true fp32 for fp32 operands: no reduced-precision tensor mode).  blockIdx.z is either a
// batch index (per-head weights: strides a_bs / w_bs / c_bs) or, with group_off != NULL, a group
// (expert) that owns rows [group_off[z], group_off[z+1]) of C, reading A through a_rows if given.
// 64x64x16 tiles, 256 threads, 4x4 outputs per thread.
// ------------------------------------------------------------------------------------------------
struct LinearArgs {
  const void* A;
  const void* W;
  void* C;
  const float* bias;
  const int32_t* a_rows;
  const int32_t* group_off;
  long long a_bs, w_bs, c_bs;
  int lda, ldc, M, N, K;
};

template <typename T, typename TC>
__global__ void __launch_bounds__(256) linear_kernel(LinearArgs a) {
  constexpr int BM = 64, BN = 64, BK = 16, LD = 68;
  __shared__ __align__(16) float As[BK][LD];
  __shared__ __align__(16) float Ws[BK][LD];
  const int z = blockIdx.z;
  int m_lo = 0, m_hi = a.M;
  const T* A = (const T*)a.A;
  const T* Wm = (const T*)a.W + (long long)z * a.w_bs;
  TC* Cm = (TC*)a.C;
  if (a.group_off) {
    m_lo = a.group_off[z];
    m_hi = a.group_off[z + 1];
  } else {
    A += (long long)z * a.a_bs;
    Cm += (long long)z * a.c_bs;
  }
  const int m0 = m_lo + blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (m0 >= m_hi) return;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  // each thread stages 4 elements of A and of W per k-tile: element e = tid + 256*i -> (row e/16, k e%16)
  long long a_off[4];
  long long w_off[4];
  bool a_ok[4], w_ok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = tid + 256 * i, r = e >> 4;
    const int m = m0 + r, n = n0 + r;
    a_ok[i] = m < m_hi;
    w_ok[i] = n < a.N;
    const int src = a_ok[i] ? (a.a_rows ? a.a_rows[m] : m) : 0;
    a_off[i] = (long long)src * a.lda;
    w_off[i] = (long long)(w_ok[i] ? n : 0) * a.K;
  }
  for (int k0 = 0; k0 < a.K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + 256 * i, r = e >> 4, kk = e & 15;
      const bool kin = k0 + kk < a.K;
      As[kk][r] = (a_ok[i] && kin) ? ldf(A + a_off[i] + k0 + kk) : 0.f;
      Ws[kk][r] = (w_ok[i] && kin) ? ldf(Wm + w_off[i] + k0 + kk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 wv = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= m_hi) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < a.N) stf(Cm + (long long)m * a.ldc + n, acc[i][j] + (a.bias ? a.bias[n] : 0.f));
    }
  }
}

// few outputs per row (a router, a gate): one warp per (row, OPW outputs), lanes stride over K — every SM
// gets work even when the whole product has a handful of 64 x 64 tiles (OPW = 8, or 2 when even that leaves
// most SMs without a warp: decode-sized batches).  Lane partials are summed in a fixed order that does not
// depend on OPW, so a row's result does not depend on the batch.
template <typename T, typename TC, int OPW>
__global__ void __launch_bounds__(256) skinny_linear_kernel(LinearArgs a) {
  const long long wg = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31, n_groups = (a.N + OPW - 1) / OPW;
  const long long m = wg / n_groups;
  const int n0 = (int)(wg % n_groups) * OPW;
  if (m >= a.M) return;
  const T* A = (const T*)a.A + m * a.lda;
  const T* Wm = (const T*)a.W;
  float acc[OPW];
#pragma unroll
  for (int j = 0; j < OPW; ++j) acc[j] = 0.f;
  bool vec_done = false;
  if constexpr (sizeof(T) == 2) {
    // bf16 rows whose start is 16-byte aligned: 8 elements per load
    if (a.K % 8 == 0 && a.lda % 8 == 0 && ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.W)) & 15) == 0) {
      for (int k = lane * 8; k < a.K; k += 256) {
        const uint4 av = ld_v4(A + k);
        const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
        for (int j = 0; j < OPW; ++j)
          if (n0 + j < a.N) {
            const uint4 wv = ld_nc_v4(Wm + (long long)(n0 + j) * a.K + k);
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              acc[j] = fmaf(bf16_lo(aw[e]), bf16_lo(ww[e]), acc[j]);
              acc[j] = fmaf(bf16_hi(aw[e]), bf16_hi(ww[e]), acc[j]);
            }
          }
      }
      vec_done = true;
    }
  }
  if (!vec_done)
    for (int k = lane; k < a.K; k += 32) {
      const float av = ldf(A + k);
#pragma unroll
      for (int j = 0; j < OPW; ++j)
        if (n0 + j < a.N) acc[j] = fmaf(av, ldf(Wm + (long long)(n0 + j) * a.K + k), acc[j]);
    }
#pragma unroll
  for (int j = 0; j < OPW; ++j) {
    const float v = warp_sum(acc[j]);
    if (lane == 0 && n0 + j < a.N) stf((TC*)a.C + m * a.ldc + n0 + j, v + (a.bias ? a.bias[n0 + j] : 0.f));
  }
}

// ------------------------------------------------------------------------------------------------
// latent attention, step 1 (one CTA per token).  proj = [query latent (q_rank) | kv latent (kv_rank) |
// shared rotated key part (rot_dim)] as the fused down-projection wrote it.
//   cq    = rmsnorm(query latent) * w_qn                                  -> cq [T, q_rank]
//   cache = [ rmsnorm(kv latent) * w_kvn | rotate(key part, position) ]   -> row slot_mapping[t]
// (has_kv = 0: the layer reads another layer's cache and only has the query part.)
// Pairs (2i, 2i+1) of the first rot_dims entries turn by position * freq[i]; angle and sin/cos in fp64.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(const T* __restrict__ proj, int ldp, int q_rank,
                                                          int kv_rank, int rot_dim, int rot_dims,
                                                          const double* __restrict__ freq,
                                                          const int32_t* __restrict__ positions,
                                                          const int32_t* __restrict__ slot_mapping,
                                                          const float* __restrict__ w_qn,
                                                          const float* __restrict__ w_kvn, T* __restrict__ cq,
                                                          T* __restrict__ cache, int has_kv, float eps, float mag) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const T* pr = proj + (long long)t * ldp;
  float ss = 0.f, inv;
  if (q_rank > 0) {  // q_rank 0: full-rank queries, no query latent
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
      const float v = ldf(pr + c);
      ss += v * v;
    }
    ss = block_sum(ss, red);
    inv = 1.f / sqrtf(ss / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
      stf(cq + (long long)t * q_rank + c, ldf(pr + c) * inv * w_qn[c]);
  }
  if (!has_kv) return;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  T* row = cache + (long long)slot * (kv_rank + rot_dim);
  const T* pc = pr + q_rank;
  ss = 0.f;
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
    const float v = ldf(pc + c);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  inv = 1.f / sqrtf(ss / (float)kv_rank + eps);
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) stf(row + c, ldf(pc + c) * inv * w_kvn[c]);
  const T* pk = pc + kv_rank;
  const double pos = (double)positions[t];
  for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
    double sn, cs;
    sincos(pos * freq[i], &sn, &cs);
    const float u = ldf(pk + 2 * i), v = ldf(pk + 2 * i + 1), c = (float)cs * mag, s = (float)sn * mag;
    stf(row + kv_rank + 2 * i, u * c - v * s);
    stf(row + kv_rank + 2 * i + 1, v * c + u * s);
  }
  for (int c = rot_dims + threadIdx.x; c < rot_dim; c += blockDim.x) stf(row + kv_rank + c, ldf(pk + c));
}

// step 2 (one CTA per token): the rotated part of every head's query, turned by the token's position, goes
// to its place behind the latent-space query: qa[t, h, kv_rank + j] (fp32).  q: [T, heads*(dim+rot_dim)].
template <typename T>
__global__ void __launch_bounds__(128) rope_q_kernel(const T* __restrict__ q, int heads, int dim, int rot_dim,
                                                     int rot_dims, const double* __restrict__ freq,
                                                     const int32_t* __restrict__ positions,
                                                     float* __restrict__ qa, int kv_rank, int ldq, float mag) {
  extern __shared__ float cs_sn[];  // [rot_dims/2][2]
  const int t = blockIdx.x, half = rot_dims / 2;
  const double pos = (double)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sn, cs;
    sincos(pos * freq[i], &sn, &cs);
    cs_sn[2 * i] = (float)cs * mag;
    cs_sn[2 * i + 1] = (float)sn * mag;
  }
  __syncthreads();
  const int RP = kv_rank + rot_dim;
  for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
    const int h = e / half, i = e % half;
    const T* src = q + (long long)t * ldq + (long long)h * (dim + rot_dim) + dim;
    float* dst = qa + ((long long)t * heads + h) * RP + kv_rank;
    const float u = ldf(src + 2 * i), v = ldf(src + 2 * i + 1), c = cs_sn[2 * i], s = cs_sn[2 * i + 1];
    dst[2 * i] = u * c - v * s;
    dst[2 * i + 1] = v * c + u * s;
  }
  const int rest = rot_dim - rot_dims;
  for (int e = threadIdx.x; e < heads * rest; e += blockDim.x) {
    const int h = e / rest, j = rot_dims + e % rest;
    qa[((long long)t * heads + h) * RP + kv_rank + j] = ldf(q + (long long)t * ldq + (long long)h * (dim + rot_dim) + dim + j);
  }
}

// ------------------------------------------------------------------------------------------------
// step 3: attention in the latent space.  The query of head h is qa[t,h,:] = [W_uk[h]^T q_unrotated |
// q_rotated] (kv_rank + rot_dim values), a cached row is [latent c | rotated key part], so the score is
// one dot product against the cached row and the value is the latent itself:
//     out[t,h,:] = softmax_j( scale * qa[t,h] . row_j ) . c_j      over  max(0, p-window+1) <= j <= p
// (the per-head value up-projection is applied to out afterwards).  One CTA per (token, group of 8
// heads); a chunk of 32 cached rows is staged in shared memory once and used by all 8 heads (warp =
// head, lane = key for the scores, lane = output dims for the weighted sum); online softmax in fp32.
// The chunks start at the window's first key, so the arithmetic of a token does not depend on how the
// prompt was cut or batched.  kv_rank <= 32 * LATENT_ACC (the accumulator registers of a lane).
// ------------------------------------------------------------------------------------------------
template <typename T, int LATENT_ACC>
__global__ void __launch_bounds__(256) latent_attn_kernel(const float* __restrict__ qa,
                                                          const T* __restrict__ cache,
                                                          const int32_t* __restrict__ block_table, int bt_stride,
                                                          const int32_t* __restrict__ row_seq,
                                                          const int32_t* __restrict__ positions, int heads,
                                                          int kv_rank, int rot_dim, int block_size, int window,
                                                          float scale, const T* __restrict__ gate, int ld_gate,
                                                          T* __restrict__ out) {
  extern __shared__ float sm[];
  const int RP = kv_rank + rot_dim, KS = RP + 1;
  float* qs = sm;            // [8][RP]
  float* ks = sm + 8 * RP;   // [32][RP+1]
  const int t = blockIdx.x, h0 = blockIdx.y * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = h0 + warp;
  const bool live = h < heads;
  const int p = positions[t];
  const int32_t* bt = block_table + (long long)row_seq[t] * bt_stride;
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  for (int e = threadIdx.x; e < 8 * RP; e += blockDim.x) {
    const int hh = h0 + e / RP;
    qs[e] = hh < heads ? qa[((long long)t * heads + hh) * RP + e % RP] : 0.f;
  }
  float m = -INFINITY, l = 0.f;
  float acc[LATENT_ACC];
#pragma unroll
  for (int i = 0; i < LATENT_ACC; ++i) acc[i] = 0.f;
  const float* qh = qs + warp * RP;
  for (int j0 = lo; j0 <= p; j0 += 32) {
    const int n = min(32, p + 1 - j0);
    __syncthreads();
    for (int e = threadIdx.x; e < n * RP; e += blockDim.x) {
      const int j = e / RP, d = e % RP, pos = j0 + j;
      const long long row = (long long)bt[pos / block_size] * block_size + pos % block_size;
      ks[j * KS + d] = ldf(cache + row * RP + d);
    }
    __syncthreads();
    if (!live) continue;
    float s = -INFINITY;
    if (lane < n) {
      const float* kr = ks + lane * KS;
      float dot = 0.f;
      for (int d = 0; d < RP; ++d) dot = fmaf(qh[d], kr[d], dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);  // m = -inf on the first chunk: exp(-inf) = 0
    const float pl = lane < n ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pl);
#pragma unroll
    for (int i = 0; i < LATENT_ACC; ++i) acc[i] *= corr;
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pl, j);
      const float* kr = ks + j * KS;
#pragma unroll
      for (int i = 0; i < LATENT_ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < kv_rank) acc[i] = fmaf(pj, kr[d], acc[i]);
      }
    }
    m = m_new;
  }
  if (!live) return;
  const float inv = (gate ? sigmoidf_(ldf(gate + (long long)t * ld_gate + h)) : 1.f) / l;
  T* o = out + ((long long)t * heads + h) * kv_rank;
#pragma unroll
  for (int i = 0; i < LATENT_ACC; ++i) {
    const int d = lane + 32 * i;
    if (d < kv_rank) stf(o + d, acc[i] * inv);
  }
}

// ------------------------------------------------------------------------------------------------
// latent attention on the tensor cores (bf16 cache).  One CTA (4 warps) per (token, group of 16 heads):
// the 16 heads are the M rows of mma.sync.m16n8k16 tiles and share every cached row, so a row fetched once
// serves 16 heads twice (as key [latent | rotated part] and as value [latent]).
//   * the fp32 query (already in latent space, times the score scale) is split into bf16 hi + lo parts and
//     both are multiplied with the keys: the scores keep ~16 bits of the query instead of 8;
//   * cached rows arrive in chunks of 64 keys by cp.async into a double-buffered shared-memory tile (the
//     next chunk loads while this one is multiplied); rows of a chunk past the token's position are zeros;
//   * warp w scores keys [16w, 16w+16) of the chunk, the chunk's row maxima / sums and the bf16 weights are
//     exchanged through shared memory, then warp w accumulates output dims [w R/4, (w+1) R/4) over all
//     64 keys (values read from the same tile with ldmatrix.trans); online softmax state in fp32.
// Chunks start at the first key of the token's window, so a token's arithmetic does not depend on how the
// prompt was cut or batched.  Needs kv_rank % 64 == 0, (kv_rank + rot_dim) % 16 == 0, kv_rank <= 32 * NTW.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

constexpr int LATENT_CHUNK = 64, LATENT_PLD = LATENT_CHUNK + 8;
template <int NTW>
__global__ void __launch_bounds__(128) latent_attn_mma_kernel(const float* __restrict__ qa,
                                                              const bf16* __restrict__ cache,
                                                              const int32_t* __restrict__ block_table, int bt_stride,
                                                              const int32_t* __restrict__ row_seq,
                                                              const int32_t* __restrict__ positions, int heads, int R,
                                                              int P, int block_size, int window, float scale,
                                                              const bf16* __restrict__ gate, int ld_gate,
                                                              bf16* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t smraw[];
  const int RP = R + P, LDS = RP + 8;
  bf16* qhi = reinterpret_cast<bf16*>(smraw);             // [16][LDS]
  bf16* qlo = qhi + 16 * LDS;                             // [16][LDS]
  bf16* kbuf = qlo + 16 * LDS;                            // [2][64][LDS]
  bf16* pbuf = kbuf + 2 * LATENT_CHUNK * LDS;             // [16][72]
  float* wmax = reinterpret_cast<float*>(pbuf + 16 * LATENT_PLD);  // [4][16]
  float* wsum = wmax + 64;                                // [4][16]
  const int t = blockIdx.x, h0 = blockIdx.y * 16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q4 = lane & 3;
  const int p = positions[t];
  const int32_t* bt = block_table + (long long)row_seq[t] * bt_stride;
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int nchunks = (p - lo) / LATENT_CHUNK + 1;
  const int cpr = RP / 8;  // 16-byte pieces of a cached row

  auto load_chunk = [&](int c, int buf) {
    const int j0 = lo + c * LATENT_CHUNK, n = min(LATENT_CHUNK, p + 1 - j0);
    bf16* kb = kbuf + (long long)buf * LATENT_CHUNK * LDS;
    // lane l looks up the pages of rows l and l + 32 of the chunk once (one division each); the warp then
    // walks its rows (warp, warp + 4, ...) with the row's cache index broadcast from the lane that holds it
    long long src_row[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int j = lane + 32 * k, pos = j0 + j;
      src_row[k] = j < n ? (long long)bt[pos / block_size] * block_size + pos % block_size : -1;
    }
    for (int j = warp; j < LATENT_CHUNK; j += 4) {
      const long long row = __shfl_sync(0xffffffffu, j < 32 ? src_row[0] : src_row[1], j & 31);
      bf16* dst = kb + j * LDS;
      if (row >= 0) {
        const bf16* src = cache + row * RP;
        for (int ck = lane; ck < cpr; ck += 32) cp_async16(dst + ck * 8, src + ck * 8);
      } else {
        for (int ck = lane; ck < cpr; ck += 32) *reinterpret_cast<uint4*>(dst + ck * 8) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
  };

  load_chunk(0, 0);
  for (int e = tid; e < 16 * RP; e += 128) {
    const int r = e / RP, d = e % RP, hh = h0 + r;
    const float v = hh < heads ? qa[((long long)t * heads + hh) * RP + d] * scale : 0.f;
    const bf16 hi = __float2bfloat16_rn(v);
    qhi[r * LDS + d] = hi;
    qlo[r * LDS + d] = __float2bfloat16_rn(v - __bfloat162float(hi));
  }
  const uint32_t qhi_s = smem_u32(qhi), qlo_s = smem_u32(qlo), p_s = smem_u32(pbuf);
  const uint32_t a_off = (uint32_t)(((lane & 15) * LDS + (lane >> 4) * 8) * 2);
  const uint32_t kq_off = (uint32_t)(((16 * warp + (lane & 7) + 8 * (lane >> 4)) * LDS + 8 * ((lane >> 3) & 1)) * 2);
  const uint32_t pa_off = (uint32_t)(((lane & 15) * LATENT_PLD + (lane >> 4) * 8) * 2);
  const int ntw = R / 32, dim_w = warp * (R / 4);
  float m_[2] = {-INFINITY, -INFINITY}, l_[2] = {0.f, 0.f};
  float o[NTW][4];
#pragma unroll
  for (int i = 0; i < NTW; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int c = 0; c < nchunks; ++c) {
    const int buf = c & 1;
    cp_async_wait_all();
    __syncthreads();  // chunk c (and, first time, the query) is in shared memory; chunk c-1 is done with
    if (c + 1 < nchunks) load_chunk(c + 1, buf ^ 1);
    const int n = min(LATENT_CHUNK, p + 1 - (lo + c * LATENT_CHUNK));
    const uint32_t kb_s = smem_u32(kbuf + (long long)buf * LATENT_CHUNK * LDS);
    // ---- scores of this warp's 16 keys: S = (Qhi + Qlo) K^T ----
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    for (int ks = 0; ks < RP / 16; ++ks) {
      uint32_t a0, a1, a2, a3, c0, c1, c2, c3, b0, b1, b2, b3;
      ldsm_x4(qhi_s + a_off + ks * 32, a0, a1, a2, a3);
      ldsm_x4(qlo_s + a_off + ks * 32, c0, c1, c2, c3);
      ldsm_x4(kb_s + kq_off + ks * 32, b0, b1, b2, b3);
      mma_bf16_16816(s[0], a0, a1, a2, a3, b0, b1);
      mma_bf16_16816(s[1], a0, a1, a2, a3, b2, b3);
      mma_bf16_16816(s[0], c0, c1, c2, c3, b0, b1);
      mma_bf16_16816(s[1], c0, c1, c2, c3, b2, b3);
    }
    // ---- online softmax over the chunk: rows g and g + 8 of this thread ----
    float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = 16 * warp + nt * 8 + 2 * q4 + (e & 1);
        if (key >= n) s[nt][e] = -INFINITY;
        rmax[e >> 1] = fmaxf(rmax[e >> 1], s[nt][e]);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 1));
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 2));
      if (q4 == 0) wmax[warp * 16 + g + 8 * r] = rmax[r];
    }
    __syncthreads();
    float corr[2], psum[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      const float cm = fmaxf(fmaxf(wmax[row], wmax[16 + row]), fmaxf(wmax[32 + row], wmax[48 + row]));
      const float mn = fmaxf(m_[r], cm);
      corr[r] = expf(m_[r] - mn);
      m_[r] = mn;
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      // the weights as the value product will see them (bf16): the row sum is taken over the same
      // rounded values, so the weights of a row still add up to one
      const float p0 = round_bf16(expf(s[nt][0] - m_[0])), p1 = round_bf16(expf(s[nt][1] - m_[0]));
      const float p2 = round_bf16(expf(s[nt][2] - m_[1])), p3 = round_bf16(expf(s[nt][3] - m_[1]));
      psum[0] += p0 + p1;
      psum[1] += p2 + p3;
      const int col = 16 * warp + nt * 8 + 2 * q4;
      *reinterpret_cast<uint32_t*>(pbuf + g * LATENT_PLD + col) = pack_bf16x2(p0, p1);
      *reinterpret_cast<uint32_t*>(pbuf + (g + 8) * LATENT_PLD + col) = pack_bf16x2(p2, p3);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
      if (q4 == 0) wsum[warp * 16 + g + 8 * r] = psum[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      l_[r] = l_[r] * corr[r] + ((wsum[row] + wsum[16 + row]) + (wsum[32 + row] + wsum[48 + row]));
    }
    // ---- output dims of this warp: O = O * corr + P V ----
#pragma unroll
    for (int i = 0; i < NTW; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < LATENT_CHUNK / 16; ++kk) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(p_s + pa_off + kk * 32, a0, a1, a2, a3);
      const int key = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const uint32_t v_row = kb_s + (uint32_t)((key * LDS + dim_w + 8 * (lane >> 4)) * 2);
#pragma unroll
      for (int nd2 = 0; nd2 < NTW / 2; ++nd2) {
        if (2 * nd2 < ntw) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(v_row + nd2 * 32, b0, b1, b2, b3);
          mma_bf16_16816(o[2 * nd2], a0, a1, a2, a3, b0, b1);
          mma_bf16_16816(o[2 * nd2 + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
  }
  float inv[2] = {1.f / l_[0], 1.f / l_[1]};
  if (gate) {  // one sigmoid gate number per head
#pragma unroll
    for (int r = 0; r < 2; ++r)
      if (h0 + g + 8 * r < heads) inv[r] *= sigmoidf_(ldf(gate + (long long)t * ld_gate + h0 + g + 8 * r));
  }
#pragma unroll
  for (int i = 0; i < NTW; ++i) {
    if (i < ntw) {
      const int dim = dim_w + i * 8 + 2 * q4;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int hh = h0 + g + 8 * r;
        if (hh < heads)
          *reinterpret_cast<uint32_t*>(out + ((long long)t * heads + hh) * R + dim) =
              pack_bf16x2(o[i][2 * r] * inv[r], o[i][2 * r + 1] * inv[r]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// The same product with the query fragments held in REGISTERS (sizes with (kv_rank + rot_dim) % 64 == 0):
// warp w owns a quarter of the key dimensions, keeps the hi / lo fragments of the 16 heads' queries for
// that quarter for the whole kernel (KS k-steps), and scores all 64 keys of a chunk over its quarter; the
// four partial score tiles are summed through shared memory in a fixed order, after which every warp holds
// the full 16 x 64 score tile in accumulator layout — softmax and the bf16 weights need no further
// exchange and feed the value product of the warp's output slice directly.  Against the kernel above:
// a third of the ldmatrix traffic (the query is never re-read), two barriers per chunk instead of three.
// ------------------------------------------------------------------------------------------------
template <int NTW, int KS>
__global__ void __launch_bounds__(128) latent_attn_mma2_kernel(const float* __restrict__ qa,
                                                               const bf16* __restrict__ cache,
                                                               const int32_t* __restrict__ block_table, int bt_stride,
                                                               const int32_t* __restrict__ row_seq,
                                                               const int32_t* __restrict__ positions, int heads, int R,
                                                               int P, int block_size, int window, float scale,
                                                               const bf16* __restrict__ gate, int ld_gate,
                                                               bf16* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t smraw[];
  const int RP = R + P, LDS = RP + 8;
  bf16* kbuf = reinterpret_cast<bf16*>(smraw);                                  // [2][64][LDS]
  float* spart = reinterpret_cast<float*>(kbuf + 2 * LATENT_CHUNK * LDS);      // [4 warps][8 n-tiles][32 lanes][4]
  bf16* qhi = kbuf + LATENT_CHUNK * LDS;                                        // staging in buffer 1: [16][LDS] x 2
  bf16* qlo = qhi + 16 * LDS;
  const int t = blockIdx.x, h0 = blockIdx.y * 16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q4 = lane & 3;
  const int p = positions[t];
  const int32_t* bt = block_table + (long long)row_seq[t] * bt_stride;
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int nchunks = (p - lo) / LATENT_CHUNK + 1;
  const int cpr = RP / 8;

  auto load_chunk = [&](int c, int buf) {
    const int j0 = lo + c * LATENT_CHUNK, n = min(LATENT_CHUNK, p + 1 - j0);
    bf16* kb = kbuf + (long long)buf * LATENT_CHUNK * LDS;
    long long src_row[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int j = lane + 32 * k, pos = j0 + j;
      src_row[k] = j < n ? (long long)bt[pos / block_size] * block_size + pos % block_size : -1;
    }
    for (int j = warp; j < LATENT_CHUNK; j += 4) {
      const long long row = __shfl_sync(0xffffffffu, j < 32 ? src_row[0] : src_row[1], j & 31);
      bf16* dst = kb + j * LDS;
      if (row >= 0) {
        const bf16* src = cache + row * RP;
        for (int ck = lane; ck < cpr; ck += 32) cp_async16(dst + ck * 8, src + ck * 8);
      } else {
        for (int ck = lane; ck < cpr; ck += 32) *reinterpret_cast<uint4*>(dst + ck * 8) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
  };

  load_chunk(0, 0);
  for (int e = tid; e < 16 * RP; e += 128) {
    const int r = e / RP, d = e % RP, hh = h0 + r;
    const float v = hh < heads ? qa[((long long)t * heads + hh) * RP + d] * scale : 0.f;
    const bf16 hi = __float2bfloat16_rn(v);
    qhi[r * LDS + d] = hi;
    qlo[r * LDS + d] = __float2bfloat16_rn(v - __bfloat162float(hi));
  }
  __syncthreads();
  uint32_t qh[KS][4], ql[KS][4];
  {
    const uint32_t a_off = (uint32_t)(((lane & 15) * LDS + (lane >> 4) * 8 + warp * KS * 16) * 2);
    const uint32_t qhi_s = smem_u32(qhi), qlo_s = smem_u32(qlo);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      ldsm_x4(qhi_s + a_off + ks * 32, qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3]);
      ldsm_x4(qlo_s + a_off + ks * 32, ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3]);
    }
  }
  const uint32_t kq_off = (uint32_t)((((lane & 7) + 8 * (lane >> 4)) * LDS + warp * KS * 16 + 8 * ((lane >> 3) & 1)) * 2);
  const int ntw = R / 32, dim_w = warp * (R / 4);
  float m_[2] = {-INFINITY, -INFINITY}, l_[2] = {0.f, 0.f};
  float o[NTW][4];
#pragma unroll
  for (int i = 0; i < NTW; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int c = 0; c < nchunks; ++c) {
    const int buf = c & 1;
    cp_async_wait_all();
    __syncthreads();  // chunk c has landed; buffer buf^1 (first time: the query staging) and spart are free
    if (c + 1 < nchunks) load_chunk(c + 1, buf ^ 1);
    const int n = min(LATENT_CHUNK, p + 1 - (lo + c * LATENT_CHUNK));
    const uint32_t kb_s = smem_u32(kbuf + (long long)buf * LATENT_CHUNK * LDS);
    // ---- partial scores of all 64 keys over this warp's quarter of the dimensions ----
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {  // k-step outside: eight independent accumulator chains per pass
      uint32_t b[4][4];
#pragma unroll
      for (int nt2 = 0; nt2 < 4; ++nt2)
        ldsm_x4(kb_s + kq_off + (uint32_t)(nt2 * 16 * LDS * 2 + ks * 32), b[nt2][0], b[nt2][1], b[nt2][2], b[nt2][3]);
#pragma unroll
      for (int nt2 = 0; nt2 < 4; ++nt2) {
        mma_bf16_16816(s[2 * nt2], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], b[nt2][0], b[nt2][1]);
        mma_bf16_16816(s[2 * nt2 + 1], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], b[nt2][2], b[nt2][3]);
      }
#pragma unroll
      for (int nt2 = 0; nt2 < 4; ++nt2) {
        mma_bf16_16816(s[2 * nt2], ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], b[nt2][0], b[nt2][1]);
        mma_bf16_16816(s[2 * nt2 + 1], ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], b[nt2][2], b[nt2][3]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
      *reinterpret_cast<float4*>(spart + ((warp * 8 + nt) * 32 + lane) * 4) = make_float4(s[nt][0], s[nt][1], s[nt][2], s[nt][3]);
    __syncthreads();
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float4 a = *reinterpret_cast<const float4*>(spart + ((0 * 8 + nt) * 32 + lane) * 4);
      const float4 b = *reinterpret_cast<const float4*>(spart + ((1 * 8 + nt) * 32 + lane) * 4);
      const float4 cc = *reinterpret_cast<const float4*>(spart + ((2 * 8 + nt) * 32 + lane) * 4);
      const float4 d = *reinterpret_cast<const float4*>(spart + ((3 * 8 + nt) * 32 + lane) * 4);
      s[nt][0] = (a.x + b.x) + (cc.x + d.x);
      s[nt][1] = (a.y + b.y) + (cc.y + d.y);
      s[nt][2] = (a.z + b.z) + (cc.z + d.z);
      s[nt][3] = (a.w + b.w) + (cc.w + d.w);
    }
    // ---- online softmax, rows g and g + 8, all 64 keys in this thread's quad ----
    float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = nt * 8 + 2 * q4 + (e & 1);
        if (key >= n) s[nt][e] = -INFINITY;
        rmax[e >> 1] = fmaxf(rmax[e >> 1], s[nt][e]);
      }
    float corr[2], psum[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 1));
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 2));
      const float mn = fmaxf(m_[r], rmax[r]);
      corr[r] = expf(m_[r] - mn);
      m_[r] = mn;
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      // rounded to what the value product sees (bf16), so that a row's weights still add up to one
      s[nt][0] = round_bf16(expf(s[nt][0] - m_[0]));
      s[nt][1] = round_bf16(expf(s[nt][1] - m_[0]));
      s[nt][2] = round_bf16(expf(s[nt][2] - m_[1]));
      s[nt][3] = round_bf16(expf(s[nt][3] - m_[1]));
      psum[0] += s[nt][0] + s[nt][1];
      psum[1] += s[nt][2] + s[nt][3];
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
      l_[r] = l_[r] * corr[r] + psum[r];
    }
    // ---- output dims of this warp: O = O * corr + P V ----
#pragma unroll
    for (int i = 0; i < NTW; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < LATENT_CHUNK / 16; ++kk) {
      const uint32_t a0 = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                     a3 = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      const int key = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const uint32_t v_row = kb_s + (uint32_t)((key * LDS + dim_w + 8 * (lane >> 4)) * 2);
#pragma unroll
      for (int nd2 = 0; nd2 < NTW / 2; ++nd2) {
        if (2 * nd2 < ntw) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(v_row + nd2 * 32, b0, b1, b2, b3);
          mma_bf16_16816(o[2 * nd2], a0, a1, a2, a3, b0, b1);
          mma_bf16_16816(o[2 * nd2 + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
  }
  float inv[2] = {1.f / l_[0], 1.f / l_[1]};
  if (gate) {  // one sigmoid gate number per head
#pragma unroll
    for (int r = 0; r < 2; ++r)
      if (h0 + g + 8 * r < heads) inv[r] *= sigmoidf_(ldf(gate + (long long)t * ld_gate + h0 + g + 8 * r));
  }
#pragma unroll
  for (int i = 0; i < NTW; ++i) {
    if (i < ntw) {
      const int dim = dim_w + i * 8 + 2 * q4;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int hh = h0 + g + 8 * r;
        if (hh < heads)
          *reinterpret_cast<uint32_t*>(out + ((long long)t * heads + hh) * R + dim) =
              pack_bf16x2(o[i][2 * r] * inv[r], o[i][2 * r + 1] * inv[r]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// generalized delta rule.  One CTA per (sequence, head), thread j owns column j of the state S[key][value]
// (kept in shared memory for the tokens of this step, loaded from / stored to the sequence's fp32 state
// slot; a sequence whose first token this step is position 0 starts from zero, whatever the slot held).
// proj row = [r | k | v | g | a | z] (heads*dim each, z = decay_rank).  Per token, per head:
//   decay w_i = exp(-e^-1/2 * sigmoid(w0_i + sum_r w2[i,r] tanh(z_r))),  a_i = sigmoid(a_i + a_bias_i),
//   u = k / sqrt(sum k^2 + 1e-6)
//   S <- diag(w) S - (a*u) (u^T S) + k v^T          (both terms read the old S)
//   o = S^T r;  out = o / sqrt(mean(o^2) + eps) * out_norm * sigmoid(g)
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void delta_rule_kernel(const T* __restrict__ proj, int ldp, const T* __restrict__ w2,
                                  const float* __restrict__ w0, const float* __restrict__ a_bias,
                                  const float* __restrict__ out_norm, float* __restrict__ state,
                                  long long slot_stride, const int32_t* __restrict__ seq_desc, int heads, int D,
                                  int Rk, float eps, T* __restrict__ out) {
  extern __shared__ float sm[];
  float* S = sm;                  // [D][D]
  float* kv_ = S + D * D;         // k
  float* us = kv_ + D;            // unit key
  float* aus = us + D;            // a * u
  float* wd = aus + D;            // decay
  float* rs = wd + D;             // receptance
  float* w2s = rs + D;            // [Rk][D]
  float* zt = w2s + (long long)Rk * D;  // [Rk]
  float* red = zt + Rk;           // [32]
  const int seq = blockIdx.x, h = blockIdx.y, i = threadIdx.x;
  const int row0 = seq_desc[4 * seq + 0], n = seq_desc[4 * seq + 1], pos0 = seq_desc[4 * seq + 2],
            slot = seq_desc[4 * seq + 3];
  const int HD = heads * D, c = h * D + i;
  const bool on = i < D;
  float* st = state + (long long)slot * slot_stride + (long long)h * D * D;
  for (int e = i; e < D * D; e += blockDim.x) S[e] = pos0 > 0 ? st[e] : 0.f;
  for (int e = i; e < Rk * D; e += blockDim.x) {
    const int r = e / D, ch = e % D;
    w2s[e] = ldf(w2 + (long long)(h * D + ch) * Rk + r);
  }
  const float w0c = on ? w0[c] : 0.f, abc = on ? a_bias[c] : 0.f, onc = on ? out_norm[c] : 0.f;
  for (int tt = 0; tt < n; ++tt) {
    const T* pr = proj + (long long)(row0 + tt) * ldp;
    for (int r = i; r < Rk; r += blockDim.x) zt[r] = tanhf(ldf(pr + 5 * HD + r));
    __syncthreads();
    float kk = 0.f, wv = 0.f, av = 0.f, rv = 0.f;
    if (on) {
      kk = ldf(pr + HD + c);
      rv = ldf(pr + c);
      float z = w0c;
      for (int r = 0; r < Rk; ++r) z = fmaf(w2s[r * D + i], zt[r], z);
      wv = expf(-0.6065306597126334f * sigmoidf_(z));
      av = sigmoidf_(ldf(pr + 4 * HD + c) + abc);
    }
    const float ssk = block_sum(kk * kk, red);
    if (on) {
      const float uu = kk / sqrtf(ssk + 1e-6f);
      kv_[i] = kk;
      us[i] = uu;
      aus[i] = av * uu;
      wd[i] = wv;
      rs[i] = rv;
    }
    __syncthreads();
    float o = 0.f;
    if (on) {
      const float vj = ldf(pr + 2 * HD + c);
      float uS = 0.f;
      for (int q = 0; q < D; ++q) uS = fmaf(us[q], S[q * D + i], uS);
      for (int q = 0; q < D; ++q) {
        const float s = wd[q] * S[q * D + i] - aus[q] * uS + kv_[q] * vj;
        S[q * D + i] = s;
        o = fmaf(s, rs[q], o);
      }
    }
    const float sso = block_sum(o * o, red);
    if (on) {
      const float y = o / sqrtf(sso / (float)D + eps) * onc * sigmoidf_(ldf(pr + 3 * HD + c));
      stf(out + (long long)(row0 + tt) * HD + c, y);
    }
  }
  __syncthreads();
  for (int e = i; e < D * D; e += blockDim.x) st[e] = S[e];
}

// The same recurrence with the state column of every thread in REGISTERS (D known at compile time): the
// per-token loops are pure FMA chains against broadcast reads of the token's vectors, no shared-memory
// traffic for S.  Used for D = 32, 64, 128; other sizes take delta_rule_kernel.
template <typename T, int D>
__global__ void __launch_bounds__(D) delta_rule_reg_kernel(const T* __restrict__ proj, int ldp, const T* __restrict__ w2,
                                                           const float* __restrict__ w0,
                                                           const float* __restrict__ a_bias,
                                                           const float* __restrict__ out_norm,
                                                           float* __restrict__ state, long long slot_stride,
                                                           const int32_t* __restrict__ seq_desc, int heads, int Rk,
                                                           float eps, T* __restrict__ out) {
  extern __shared__ float sm[];
  float* kv_ = sm;                // k
  float* us = kv_ + D;            // unit key
  float* aus = us + D;            // a * u
  float* wd = aus + D;            // decay
  float* rs = wd + D;             // receptance
  float* w2s = rs + D;            // [Rk][D+1]
  float* zt = w2s + (long long)Rk * (D + 1);  // [Rk]
  float* red = zt + Rk;           // [32]
  const int seq = blockIdx.x, h = blockIdx.y, i = threadIdx.x;
  const int row0 = seq_desc[4 * seq + 0], n = seq_desc[4 * seq + 1], pos0 = seq_desc[4 * seq + 2],
            slot = seq_desc[4 * seq + 3];
  const int HD = heads * D, c = h * D + i;
  float* st = state + (long long)slot * slot_stride + (long long)h * D * D;
  float S[D];
#pragma unroll
  for (int q = 0; q < D; ++q) S[q] = pos0 > 0 ? st[q * D + i] : 0.f;
  for (int e = i; e < Rk * D; e += D) {  // coalesced over the inner (rank) index of w2 [HD, Rk]
    const int ch = e / Rk, r = e % Rk;
    w2s[r * (D + 1) + ch] = ldf(w2 + (long long)(h * D + ch) * Rk + r);
  }
  const float w0c = w0[c], abc = a_bias[c], onc = out_norm[c];
  for (int tt = 0; tt < n; ++tt) {
    const T* pr = proj + (long long)(row0 + tt) * ldp;
    for (int r = i; r < Rk; r += D) zt[r] = tanhf(ldf(pr + 5 * HD + r));
    const float kk = ldf(pr + HD + c), rv = ldf(pr + c), vj = ldf(pr + 2 * HD + c);
    const float av = sigmoidf_(ldf(pr + 4 * HD + c) + abc), gv = sigmoidf_(ldf(pr + 3 * HD + c));
    const float ssk = block_sum(kk * kk, red);  // (its barriers also publish zt)
    float z = w0c;
    for (int r = 0; r < Rk; ++r) z = fmaf(w2s[r * (D + 1) + i], zt[r], z);
    const float uu = kk / sqrtf(ssk + 1e-6f);
    kv_[i] = kk;
    us[i] = uu;
    aus[i] = av * uu;
    wd[i] = expf(-0.6065306597126334f * sigmoidf_(z));
    rs[i] = rv;
    __syncthreads();
    float uS = 0.f;
#pragma unroll
    for (int q = 0; q < D; ++q) uS = fmaf(us[q], S[q], uS);
    float o = 0.f;
#pragma unroll
    for (int q = 0; q < D; ++q) {
      S[q] = wd[q] * S[q] - aus[q] * uS + kv_[q] * vj;
      o = fmaf(S[q], rs[q], o);
    }
    const float sso = block_sum(o * o, red);  // (its barriers keep the next token's writes behind these reads)
    stf(out + (long long)(row0 + tt) * HD + c, o / sqrtf(sso / (float)D + eps) * onc * gv);
  }
#pragma unroll
  for (int q = 0; q < D; ++q) st[q * D + i] = S[q];
}

// ------------------------------------------------------------------------------------------------
// The delta rule in three launches (D = 32, 64, 128).  Everything that does not depend on the state is
// computed for all tokens at once, so the sequential kernel is a bare chain of FMAs on a register-resident
// state column with no barrier per token:
//   prepare   (CTA per token x head): vec[t,h] = {k, u, a*u, w, r}  (fp32, 5 x D)
//   recur     (CTA per sequence x head, thread j = value column j): S <- diag(w) S - (a*u)(u^T S) + k v_j,
//             o_j = sum_q S[q] r[q]  -> raw[t, h*D + j] (fp32)
//   finish    (CTA per token x head): out = raw / rms(raw) * out_norm * sigmoid(g)
// ------------------------------------------------------------------------------------------------
constexpr int DELTA_PREP_TOKENS = 16;  // tokens per CTA of the prepare kernel: the head's decay matrix is staged once
template <typename T>
__global__ void delta_prepare_kernel(const T* __restrict__ proj, int ldp, const T* __restrict__ w2,
                                     const float* __restrict__ w0, const float* __restrict__ a_bias, int heads, int D,
                                     int Rk, int Tn, float* __restrict__ vec) {
  extern __shared__ float sm[];
  float* w2s = sm;                           // [Rk][D+1]
  float* zt = w2s + (long long)Rk * (D + 1); // [Rk]
  float* red = zt + Rk;                      // [32]
  const int h = blockIdx.y, i = threadIdx.x, HD = heads * D, c = h * D + i;
  for (int e = i; e < Rk * D; e += blockDim.x) {  // coalesced over the inner (rank) index of w2 [HD, Rk]
    const int ch = e / Rk, r = e % Rk;
    w2s[r * (D + 1) + ch] = ldf(w2 + (long long)(h * D + ch) * Rk + r);
  }
  const float w0c = w0[c], abc = a_bias[c];
  const int t_end = min(Tn, (int)(blockIdx.x + 1) * DELTA_PREP_TOKENS);
  for (int t = blockIdx.x * DELTA_PREP_TOKENS; t < t_end; ++t) {
    const T* pr = proj + (long long)t * ldp;
    __syncthreads();  // the previous token's zt has been read (first time: w2s is complete)
    for (int r = i; r < Rk; r += blockDim.x) zt[r] = tanhf(ldf(pr + 5 * HD + r));
    const float kk = ldf(pr + HD + c);
    const float ssk = block_sum(kk * kk, red);  // (its barriers also publish zt)
    float z = w0c;
    for (int r = 0; r < Rk; ++r) z = fmaf(w2s[r * (D + 1) + i], zt[r], z);
    const float uu = kk / sqrtf(ssk + 1e-6f);
    float* o = vec + ((long long)t * heads + h) * 5 * D;
    o[i] = kk;
    o[D + i] = uu;
    o[2 * D + i] = sigmoidf_(ldf(pr + 4 * HD + c) + abc) * uu;
    o[3 * D + i] = expf(-0.6065306597126334f * sigmoidf_(z));
    o[4 * D + i] = ldf(pr + c);
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(D) delta_recur_kernel(const T* __restrict__ proj, int ldp,
                                                        const float* __restrict__ vec, float* __restrict__ state,
                                                        long long slot_stride, const int32_t* __restrict__ seq_desc,
                                                        int heads, float* __restrict__ raw) {
  // the per-token vectors of DELTA_G tokens at a time come into shared memory by cp.async, one group ahead
  // of the one being consumed, so the chain below never waits for global memory
  constexpr int G = 8, TOK = 5 * D;                 // floats per token
  __shared__ __align__(16) float sv[2][G][TOK];
  const int seq = blockIdx.x, h = blockIdx.y, i = threadIdx.x;
  const int row0 = seq_desc[4 * seq + 0], n = seq_desc[4 * seq + 1], pos0 = seq_desc[4 * seq + 2],
            slot = seq_desc[4 * seq + 3];
  const int HD = heads * D, c = h * D + i;
  float* st = state + (long long)slot * slot_stride + (long long)h * D * D;
  auto fetch = [&](int g0, int buf) {
    const int cnt = min(G, n - g0);
    for (int e = i; e < cnt * (TOK / 4); e += D) {
      const int tt = e / (TOK / 4), pc = e % (TOK / 4);
      cp_async16(&sv[buf][tt][pc * 4], vec + ((long long)(row0 + g0 + tt) * heads + h) * TOK + pc * 4);
    }
    cp_async_commit();
  };
  fetch(0, 0);
  float S[D];
#pragma unroll
  for (int q = 0; q < D; ++q) S[q] = pos0 > 0 ? st[q * D + i] : 0.f;
  for (int g0 = 0, buf = 0; g0 < n; g0 += G, buf ^= 1) {
    const int cnt = min(G, n - g0);
    float vj[G];
#pragma unroll
    for (int tt = 0; tt < G; ++tt)
      vj[tt] = tt < cnt ? ldf(proj + (long long)(row0 + g0 + tt) * ldp + 2 * HD + c) : 0.f;
    cp_async_wait_all();
    __syncthreads();  // this group has landed; the other buffer is no longer read
    if (g0 + G < n) fetch(g0 + G, buf ^ 1);
#pragma unroll
    for (int tt = 0; tt < G; ++tt) {
      if (tt < cnt) {
        const float4* v4 = reinterpret_cast<const float4*>(&sv[buf][tt][0]);
        float u0 = 0.f, u1 = 0.f, u2 = 0.f, u3 = 0.f;
#pragma unroll
        for (int q = 0; q < D / 4; ++q) {
          const float4 u = v4[D / 4 + q];
          u0 = fmaf(u.x, S[4 * q], u0);
          u1 = fmaf(u.y, S[4 * q + 1], u1);
          u2 = fmaf(u.z, S[4 * q + 2], u2);
          u3 = fmaf(u.w, S[4 * q + 3], u3);
        }
        const float uS = (u0 + u1) + (u2 + u3), vv = vj[tt];
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int q = 0; q < D / 4; ++q) {
          const float4 k = v4[q], au = v4[2 * (D / 4) + q], w = v4[3 * (D / 4) + q], r = v4[4 * (D / 4) + q];
          S[4 * q] = w.x * S[4 * q] - au.x * uS + k.x * vv;
          S[4 * q + 1] = w.y * S[4 * q + 1] - au.y * uS + k.y * vv;
          S[4 * q + 2] = w.z * S[4 * q + 2] - au.z * uS + k.z * vv;
          S[4 * q + 3] = w.w * S[4 * q + 3] - au.w * uS + k.w * vv;
          o0 = fmaf(S[4 * q], r.x, o0);
          o1 = fmaf(S[4 * q + 1], r.y, o1);
          o2 = fmaf(S[4 * q + 2], r.z, o2);
          o3 = fmaf(S[4 * q + 3], r.w, o3);
        }
        raw[(long long)(row0 + g0 + tt) * HD + c] = (o0 + o1) + (o2 + o3);
      }
    }
  }
#pragma unroll
  for (int q = 0; q < D; ++q) st[q * D + i] = S[q];
}

template <typename T>
__global__ void delta_finish_kernel(const float* __restrict__ raw, const T* __restrict__ proj, int ldp,
                                    const float* __restrict__ out_norm, int heads, int D, float eps,
                                    T* __restrict__ out) {
  __shared__ float red[32];
  const int t = blockIdx.x, h = blockIdx.y, i = threadIdx.x, HD = heads * D, c = h * D + i;
  const float o = raw[(long long)t * HD + c];
  const float sso = block_sum(o * o, red);
  const float gv = sigmoidf_(ldf(proj + (long long)t * ldp + 3 * HD + c));
  stf(out + (long long)t * HD + c, o / sqrtf(sso / (float)D + eps) * out_norm[c] * gv);
}

// ------------------------------------------------------------------------------------------------
// PolyNorm: y = a N(z) + b N(z^2) + c N(z^3) + e, N(v) = v / sqrt(mean(v^2) + eps) over the row
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) polynorm_kernel(const T* __restrict__ z, const float* __restrict__ coef,
                                                       T* __restrict__ y, int F, float eps) {
  __shared__ float red[32];
  const T* zr = z + (long long)blockIdx.x * F;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int c = threadIdx.x; c < F; c += blockDim.x) {
    const float v = ldf(zr + c), v2 = v * v;
    s2 += v2;
    s4 += v2 * v2;
    s6 += v2 * v2 * v2;
  }
  s2 = block_sum(s2, red);
  s4 = block_sum(s4, red);
  s6 = block_sum(s6, red);
  const float i1 = coef[0] / sqrtf(s2 / (float)F + eps), i2 = coef[1] / sqrtf(s4 / (float)F + eps),
              i3 = coef[2] / sqrtf(s6 / (float)F + eps), e = coef[3];
  for (int c = threadIdx.x; c < F; c += blockDim.x) {
    const float v = ldf(zr + c);
    stf(y + (long long)blockIdx.x * F + c, v * i1 + v * v * i2 + v * v * v * i3 + e);
  }
}

// clamped gated unit: gu = [gate (F) | up (F)] per row; y = g' sigmoid(1.702 g') (u' + 1),
// g' = min(g, limit), u' = clamp(u, -limit, limit)
template <typename T>
__global__ void __launch_bounds__(256) clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ y,
                                                          long long rows, int F, float limit) {
  const long long total = rows * F;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const long long r = e / F;
    const int c = (int)(e % F);
    const float g = fminf(ldf(gu + r * 2 * F + c), limit);
    const float u = fminf(fmaxf(ldf(gu + r * 2 * F + F + c), -limit), limit);
    stf(y + e, g * sigmoidf_(1.702f * g) * (u + 1.f));
  }
}

// ------------------------------------------------------------------------------------------------
// top-k routing: one warp per token over fp32 router logits [T, E]; the k largest (ties: lowest index),
// weights = softmax over the chosen logits.  k <= 32.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int Tn, int E, int top,
                                                        int score_mode, int32_t* __restrict__ idx,
                                                        float* __restrict__ wts) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= Tn) return;
  const float* z = logits + (long long)t * E;
  float chosen_v = 0.f;  // lane k keeps the k-th choice
  int chosen_i = -1;
  float prev_v = INFINITY;
  int prev_i = -1;
  for (int k = 0; k < top; ++k) {
    // the largest (value, -index) strictly below the previous choice in that order
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      const bool below = v < prev_v || (v == prev_v && e > prev_i);
      if (below && (v > bv || (v == bv && e < bi))) {
        bv = v;
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == k) {
      chosen_v = bv;
      chosen_i = bi;
    }
    prev_v = bv;
    prev_i = bi;
  }
  const float top_v = __shfl_sync(0xffffffffu, chosen_v, 0);
  const float ex = lane < top ? expf(chosen_v - top_v) : 0.f;
  const float sum = warp_sum(ex);
  if (lane < top) {
    idx[(long long)t * top + lane] = chosen_i;
    // score_mode 1: every chosen expert keeps its own sigmoid score (the order by logit is the order by score)
    wts[(long long)t * top + lane] = score_mode == 1 ? sigmoidf_(chosen_v) : ex / sum;
  }
}

// grouping of the (token, choice) pairs by expert for the grouped linear layers (one CTA):
// group_off[E+1], perm_tok[pos] = token of the pair at sorted position pos, pair_pos[pair] = pos.
// The order inside a group comes from atomics and may differ between runs; rows are independent, so
// no result depends on it.
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int32_t* __restrict__ idx, int P, int top, int E,
                                                        int32_t* __restrict__ group_off,
                                                        int32_t* __restrict__ perm_tok,
                                                        int32_t* __restrict__ pair_pos,
                                                        int32_t* __restrict__ tile_tab,
                                                        int32_t* __restrict__ n_tiles) {
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
    if (tile_tab) {  // the 128-row tiles of every non-empty group, for the grouped tensor-core GEMM
      int n = 0;
      for (int e = 0; e < E; ++e)
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

// ------------------------------------------------------------------------------------------------
// end of a parallel layer: x += mixer + ff, with ff either a dense branch (f) or the routed sum
//   sum_k wts[t,k] * expert_out[pair_pos[t*top+k], :]  (+ sigmoid(shared_gate[t]) * shared_out[t, :])
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) layer_sum_kernel(float* __restrict__ x, const T* __restrict__ mix,
                                                        const T* __restrict__ f, const T* __restrict__ expert_out,
                                                        const int32_t* __restrict__ pair_pos,
                                                        const float* __restrict__ wts, int top,
                                                        const T* __restrict__ shared_out,
                                                        const float* __restrict__ shared_gate, int Tn, int W) {
  const long long total = (long long)Tn * W;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(e / W), c = (int)(e % W);
    float ff = 0.f;
    if (f) ff = ldf(f + e);
    if (expert_out) {
      for (int k = 0; k < top; ++k)
        ff = fmaf(wts[(long long)t * top + k], ldf(expert_out + (long long)pair_pos[(long long)t * top + k] * W + c), ff);
      if (shared_out) ff = fmaf(sigmoidf_(shared_gate[t]), ldf(shared_out + e), ff);
    }
    x[e] += ldf(mix + e) + ff;
  }
}

// greedy sampler over fp32 logits (lowest index wins ties) and the bf16 copy the temperature sampler reads
__global__ void __launch_bounds__(256) argmax_f32_kernel(const float* __restrict__ logits, int32_t* __restrict__ ids,
                                                         int V) {
  __shared__ float bv[256];
  __shared__ int bi[256];
  const float* z = logits + (long long)blockIdx.x * V;
  float v = -INFINITY;
  int ix = 0x7fffffff;
  for (int c = threadIdx.x; c < V; c += blockDim.x)
    if (z[c] > v || (z[c] == v && c < ix)) {
      v = z[c];
      ix = c;
    }
  bv[threadIdx.x] = v;
  bi[threadIdx.x] = ix;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      const float ov = bv[threadIdx.x + o];
      const int oi = bi[threadIdx.x + o];
      if (ov > bv[threadIdx.x] || (ov == bv[threadIdx.x] && oi < bi[threadIdx.x])) {
        bv[threadIdx.x] = ov;
        bi[threadIdx.x] = oi;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) ids[blockIdx.x] = bi[0] == 0x7fffffff ? 0 : bi[0];
}
__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* __restrict__ in, bf16* __restrict__ out,
                                                          long long n) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x)
    out[e] = __float2bfloat16_rn(in[e]);
}
__global__ void __launch_bounds__(256) copy_f32_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                       long long n) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x)
    out[e] = in[e];
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_embed_f32(const int32_t* ids, const int32_t* prev_out, const void* table, float* out, int T_, int W,
                    float scale, int dtype, void* stream) {
  B200Q_CHECK_ARG(ids && table && out && T_ >= 0 && W > 0 && is_dtype(dtype), "embed_f32: bad argument");
  if (T_ == 0) return B200Q_OK;
  DISPATCH_T(dtype, (embed_f32_kernel<T><<<grid_for((long long)T_ * W), 256, 0, as_stream(stream)>>>(
                        ids, prev_out, (const T*)table, out, T_, W, scale)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_centered_rmsnorm(const float* x, const int32_t* rows, const float* w1, const float* w2, void* y1,
                           void* y2, int n, int W, float eps, int dtype, void* stream) {
  B200Q_CHECK_ARG(x && w1 && y1 && (!y2 || w2) && n >= 0 && W > 0 && is_dtype(dtype),
                  "centered_rmsnorm: bad argument");
  if (n == 0) return B200Q_OK;
  DISPATCH_T(dtype, (centered_norm_kernel<T><<<n, 256, 0, as_stream(stream)>>>(x, rows, w1, w2, (T*)y1, (T*)y2, W, eps)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// the general form behind b200q_linear / _batched / _grouped
static int launch_linear(const LinearArgs& a, int tiles_m, int nz, int dtype, int out_f32, void* stream) {
  if (tiles_m <= 0 || nz <= 0 || a.N <= 0) return B200Q_OK;
  if (nz == 1 && !a.group_off && a.N <= 64) {
    // fewer outputs per warp when 8 would leave most of the 148 SMs without a warp
    const bool narrow = (long long)a.M * ((a.N + 7) / 8) < 148 * 16;
    const int opw = narrow ? 2 : 8;
    const long long warps = (long long)a.M * ((a.N + opw - 1) / opw);
    const unsigned blocks = (unsigned)((warps + 7) / 8);
#define SKINNY(TT, TC)                                                                     \
  do {                                                                                     \
    if (narrow) skinny_linear_kernel<TT, TC, 2><<<blocks, 256, 0, as_stream(stream)>>>(a); \
    else skinny_linear_kernel<TT, TC, 8><<<blocks, 256, 0, as_stream(stream)>>>(a);        \
  } while (0)
    if (dtype == B200Q_DTYPE_F32) SKINNY(float, float);
    else if (out_f32) SKINNY(bf16, float);
    else SKINNY(bf16, bf16);
#undef SKINNY
    B200Q_LAUNCH_CHECK();
    return B200Q_OK;
  }
  dim3 grid((a.N + 63) / 64, tiles_m, nz);
  B200Q_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "linear: grid too large (rows=%d groups=%d)", a.M, nz);
  if (dtype == B200Q_DTYPE_F32) {
    linear_kernel<float, float><<<grid, 256, 0, as_stream(stream)>>>(a);
  } else if (out_f32) {
    linear_kernel<bf16, float><<<grid, 256, 0, as_stream(stream)>>>(a);
  } else {
    linear_kernel<bf16, bf16><<<grid, 256, 0, as_stream(stream)>>>(a);
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_linear(const void* A, int lda, const void* W, const float* bias, void* C, int ldc, int M, int N, int K,
                 int dtype, int out_f32, void* stream) {
  B200Q_CHECK_ARG(A && W && C && M >= 0 && N > 0 && K > 0 && lda >= K && ldc >= N && is_dtype(dtype),
                  "linear: bad argument (M=%d N=%d K=%d lda=%d ldc=%d)", M, N, K, lda, ldc);
  if (M == 0) return B200Q_OK;
  // shapes the tcgen05 GEMM takes go to the tensor cores
  if (dtype == B200Q_DTYPE_BF16 && !out_f32 && !bias && lda == K && ldc == N && K % 64 == 0 && N % 64 == 0 &&
      ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(C)) & 15) == 0)
    return b200q_gemm_bf16(A, W, C, M, N, K, stream);
  // fp32 results (logits) of bf16 operands: the same pipeline with an fp32 epilogue
  if (dtype == B200Q_DTYPE_BF16 && out_f32 && !bias && b200q_gemm_grouped_ok(A, lda, 0, W, C, ldc, 0, N, K, 1))
    return b200q_gemm_grouped_bf16(A, M, lda, 0, W, 1, C, ldc, 0, M, N, K, nullptr, nullptr, 0, 1, stream);
  LinearArgs a{A, W, C, bias, nullptr, nullptr, 0, 0, 0, lda, ldc, M, N, K};
  return launch_linear(a, (M + 63) / 64, 1, dtype, out_f32, stream);
}

int b200q_linear_batched(const void* A, int lda, long long a_bs, const void* W, long long w_bs, void* C, int ldc,
                         long long c_bs, int M, int N, int K, int batch, int dtype, int out_f32, void* stream) {
  B200Q_CHECK_ARG(A && W && C && M >= 0 && N > 0 && K > 0 && batch > 0 && is_dtype(dtype),
                  "linear_batched: bad argument");
  if (M == 0) return B200Q_OK;
  // per-head weights stacked [batch*N, K], every head a column slice of A and of C: one grouped launch
  if (dtype == B200Q_DTYPE_BF16 && w_bs == (long long)N * K && a_bs < (1 << 30) && c_bs < (1 << 30) &&
      b200q_gemm_grouped_ok(A, lda, (int)a_bs, W, C, ldc, (int)c_bs, N, K, out_f32))
    return b200q_gemm_grouped_bf16(A, M, lda, (int)a_bs, W, batch, C, ldc, (int)c_bs, M, N, K, nullptr, nullptr, 0,
                                   out_f32, stream);
  LinearArgs a{A, W, C, nullptr, nullptr, nullptr, a_bs, w_bs, c_bs, lda, ldc, M, N, K};
  return launch_linear(a, (M + 63) / 64, batch, dtype, out_f32, stream);
}

int b200q_linear_grouped(const void* A, int lda, const int32_t* a_rows, const void* W, long long w_gs, void* C,
                         int ldc, const int32_t* group_off, int groups, int max_rows, int N, int K, int dtype,
                         const void* tile_tab, const int32_t* n_tiles, void* stream) {
  B200Q_CHECK_ARG(A && W && C && group_off && groups > 0 && max_rows >= 0 && N > 0 && K > 0 && is_dtype(dtype),
                  "linear_grouped: bad argument");
  if (max_rows == 0) return B200Q_OK;
  if (dtype == B200Q_DTYPE_BF16 && tile_tab && n_tiles && !a_rows && w_gs == (long long)N * K &&
      b200q_gemm_grouped_ok(A, lda, 0, W, C, ldc, 0, N, K, 0))
    return b200q_gemm_grouped_bf16(A, max_rows, lda, 0, W, groups, C, ldc, 0, 0, N, K, tile_tab, n_tiles,
                                   max_rows / 128 + groups, 0, stream);
  LinearArgs a{A, W, C, nullptr, a_rows, group_off, 0, w_gs, 0, lda, ldc, max_rows, N, K};
  return launch_linear(a, (max_rows + 63) / 64, groups, dtype, 0, stream);
}

int b200q_latent_prep(const void* proj, int ldp, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                      const double* freq, const int32_t* positions, const int32_t* slot_mapping,
                      const float* w_qn, const float* w_kvn, void* cq, void* cache, int has_kv, int T_, float eps,
                      int dtype, void* stream) {
  B200Q_CHECK_ARG(q_rank > 0, "latent_prep: bad argument");
  return b200q_latent_prep_ex(proj, ldp, q_rank, kv_rank, rot_dim, rot_dims, freq, 1.f, positions, slot_mapping, w_qn,
                              w_kvn, cq, cache, has_kv, T_, eps, dtype, stream);
}

int b200q_latent_prep_ex(const void* proj, int ldp, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                         const double* freq, float mag, const int32_t* positions, const int32_t* slot_mapping,
                         const float* w_qn, const float* w_kvn, void* cq, void* cache, int has_kv, int T_, float eps,
                         int dtype, void* stream) {
  B200Q_CHECK_ARG(proj && positions && q_rank >= 0 && (q_rank == 0 || (w_qn && cq)) && (q_rank > 0 || has_kv) &&
                      is_dtype(dtype) && T_ >= 0,
                  "latent_prep: bad argument");
  B200Q_CHECK_ARG(!has_kv || (cache && slot_mapping && w_kvn && (freq || rot_dims == 0) && kv_rank > 0 && rot_dim >= 0 &&
                              rot_dims % 2 == 0 && rot_dims <= rot_dim),
                  "latent_prep: bad cache arguments (kv_rank=%d rot_dim=%d rot_dims=%d)", kv_rank, rot_dim, rot_dims);
  if (T_ == 0) return B200Q_OK;
  DISPATCH_T(dtype, (latent_prep_kernel<T><<<T_, 128, 0, as_stream(stream)>>>(
                        (const T*)proj, ldp, q_rank, kv_rank, rot_dim, rot_dims, freq, positions, slot_mapping, w_qn,
                        w_kvn, (T*)cq, (T*)cache, has_kv, eps, mag)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_rope_pairs_q(const void* q, int heads, int dim, int rot_dim, int rot_dims, const double* freq,
                       const int32_t* positions, float* qa, int kv_rank, int T_, int dtype, void* stream) {
  return b200q_rope_pairs_q_ex(q, heads * (dim + rot_dim), heads, dim, rot_dim, rot_dims, freq, 1.f, positions, qa, kv_rank,
                               T_, dtype, stream);
}

int b200q_rope_pairs_q_ex(const void* q, int ldq, int heads, int dim, int rot_dim, int rot_dims, const double* freq,
                          float mag, const int32_t* positions, float* qa, int kv_rank, int T_, int dtype, void* stream) {
  B200Q_CHECK_ARG(ldq >= heads * (dim + rot_dim), "rope_pairs_q: row stride %d below the heads' %d values", ldq,
                  heads * (dim + rot_dim));
  B200Q_CHECK_ARG(q && (freq || rot_dims == 0) && positions && qa && heads > 0 && dim >= 0 && rot_dims % 2 == 0 && rot_dims <= rot_dim &&
                      is_dtype(dtype) && T_ >= 0,
                  "rope_pairs_q: bad argument");
  if (T_ == 0 || rot_dim == 0) return B200Q_OK;
  DISPATCH_T(dtype, (rope_q_kernel<T><<<T_, 128, (size_t)(rot_dims + 2) * sizeof(float), as_stream(stream)>>>(
                        (const T*)q, heads, dim, rot_dim, rot_dims, freq, positions, qa, kv_rank, ldq, mag)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_latent_attn(const float* qa, const void* cache, const int32_t* block_table, int bt_stride,
                      const int32_t* row_seq, const int32_t* positions, int T_, int heads, int kv_rank, int rot_dim,
                      int block_size, int window, float scale, void* out, int dtype, void* stream) {
  return b200q_latent_attn_ex(qa, cache, block_table, bt_stride, row_seq, positions, T_, heads, kv_rank, rot_dim, block_size,
                              window, scale, nullptr, 0, out, dtype, stream);
}

int b200q_latent_attn_ex(const float* qa, const void* cache, const int32_t* block_table, int bt_stride,
                         const int32_t* row_seq, const int32_t* positions, int T_, int heads, int kv_rank, int rot_dim,
                         int block_size, int window, float scale, const void* gate, int ld_gate, void* out, int dtype,
                         void* stream) {
  B200Q_CHECK_ARG(!gate || ld_gate >= heads, "latent_attn: gate rows of stride %d hold fewer than %d heads", ld_gate, heads);
  B200Q_CHECK_ARG(qa && cache && block_table && row_seq && positions && out && heads > 0 && T_ >= 0 &&
                      block_size > 0 && window >= 0 && is_dtype(dtype),
                  "latent_attn: bad argument");
  B200Q_CHECK_ARG(kv_rank > 0 && kv_rank <= 1024, "latent_attn: kv_rank=%d unsupported (1..1024)", kv_rank);
  if (T_ == 0) return B200Q_OK;
  const int RP = kv_rank + rot_dim;
  const size_t smem = (size_t)(8 * RP + 32 * (RP + 1)) * sizeof(float);
  B200Q_CHECK_ARG(smem <= 227 * 1024, "latent_attn: kv_rank + rot_dim = %d does not fit shared memory", RP);
  // bf16 caches whose sizes fit the tensor-core tiles (B200Q_LATENT_MMA=0: the scalar kernel everywhere)
  static const char mma_mode = [] {  // 0: scalar kernel everywhere, 1: never the register-query variant
    const char* v = getenv("B200Q_LATENT_MMA");
    return v ? v[0] : '2';
  }();
  const bool use_mma = mma_mode != '0';
  if (use_mma && dtype == B200Q_DTYPE_BF16 && kv_rank % 64 == 0 && kv_rank <= 512 && RP % 16 == 0 &&
      (reinterpret_cast<uintptr_t>(cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0) {
    const int LDS = RP + 8;
    const size_t sm2 = (size_t)(32 + 2 * LATENT_CHUNK) * LDS * 2 + 16 * LATENT_PLD * 2 + 128 * sizeof(float);
    if (sm2 <= 227 * 1024) {
      dim3 grid2(T_, (heads + 15) / 16);
      // sizes whose key dimensions split evenly over the four warps keep the query in registers
      const size_t sm3 = (size_t)2 * LATENT_CHUNK * LDS * 2 + 4 * 8 * 32 * 4 * sizeof(float);
#define LATENT_MMA2(NTW, KS)                                                                                       \
  do {                                                                                                            \
    B200Q_CUDA(cudaFuncSetAttribute(latent_attn_mma2_kernel<NTW, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                    (int)sm3));                                                                   \
    latent_attn_mma2_kernel<NTW, KS><<<grid2, 128, sm3, as_stream(stream)>>>(                                      \
        qa, (const bf16*)cache, block_table, bt_stride, row_seq, positions, heads, kv_rank, rot_dim, block_size, \
        window, scale, (const bf16*)gate, ld_gate, (bf16*)out);                                                   \
    B200Q_LAUNCH_CHECK();                                                                                         \
    return B200Q_OK;                                                                                              \
  } while (0)
      if (RP % 64 == 0 && mma_mode != '1') {
        if (kv_rank == 512 && RP == 576) LATENT_MMA2(16, 9);
        if (kv_rank == 256 && RP == 320) LATENT_MMA2(8, 5);
        if (kv_rank == 128 && RP == 192) LATENT_MMA2(4, 3);
        if (kv_rank == 64 && RP == 128) LATENT_MMA2(2, 2);
      }
#undef LATENT_MMA2
#define LATENT_MMA(NTW)                                                                                           \
  do {                                                                                                            \
    B200Q_CUDA(cudaFuncSetAttribute(latent_attn_mma_kernel<NTW>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                    (int)sm2));                                                                   \
    latent_attn_mma_kernel<NTW><<<grid2, 128, sm2, as_stream(stream)>>>(                                          \
        qa, (const bf16*)cache, block_table, bt_stride, row_seq, positions, heads, kv_rank, rot_dim, block_size, \
        window, scale, (const bf16*)gate, ld_gate, (bf16*)out);                                                   \
  } while (0)
      if (kv_rank <= 128) LATENT_MMA(4);
      else if (kv_rank <= 256) LATENT_MMA(8);
      else LATENT_MMA(16);
#undef LATENT_MMA
      B200Q_LAUNCH_CHECK();
      return B200Q_OK;
    }
  }
  dim3 grid(T_, (heads + 7) / 8);
#define LATENT_LAUNCH(TT, ACC)                                                                                     \
  do {                                                                                                             \
    B200Q_CUDA(cudaFuncSetAttribute(latent_attn_kernel<TT, ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                    (int)smem));                                                                   \
    latent_attn_kernel<TT, ACC><<<grid, 256, smem, as_stream(stream)>>>(                                           \
        qa, (const TT*)cache, block_table, bt_stride, row_seq, positions, heads, kv_rank, rot_dim, block_size,    \
        window, scale, (const TT*)gate, ld_gate, (TT*)out);                                                        \
  } while (0)
#define LATENT_BY_RANK(TT)                          \
  do {                                              \
    if (kv_rank <= 128) LATENT_LAUNCH(TT, 4);       \
    else if (kv_rank <= 256) LATENT_LAUNCH(TT, 8);  \
    else if (kv_rank <= 512) LATENT_LAUNCH(TT, 16); \
    else LATENT_LAUNCH(TT, 32);                     \
  } while (0)
  if (dtype == B200Q_DTYPE_F32) LATENT_BY_RANK(float);
  else LATENT_BY_RANK(bf16);
#undef LATENT_BY_RANK
#undef LATENT_LAUNCH
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_delta_rule(const void* proj, int ldp, const void* w2, const float* w0, const float* a_bias,
                     const float* out_norm, float* state, long long slot_stride, const int32_t* seq_desc,
                     int n_seqs, int heads, int D, int Rk, float eps, void* out, int dtype, float* scratch, int T_,
                     void* stream) {
  B200Q_CHECK_ARG(proj && w2 && w0 && a_bias && out_norm && state && seq_desc && out && heads > 0 && D > 0 &&
                      Rk > 0 && n_seqs >= 0 && is_dtype(dtype),
                  "delta_rule: bad argument");
  if (n_seqs == 0) return B200Q_OK;
  if (scratch && T_ > 0 && (D == 32 || D == 64 || D == 128)) {
    // three launches: per-token vectors for all rows, the bare recurrence, norm and gate for all rows
    float* vec = scratch;
    float* raw = scratch + (long long)T_ * heads * D * 5;
    dim3 tg(T_, heads), sg(n_seqs, heads);
    cudaStream_t st = as_stream(stream);
    const size_t psm = ((size_t)Rk * (D + 1) + Rk + 32) * sizeof(float);
    B200Q_CHECK_ARG(psm <= 227 * 1024, "delta_rule: decay rank %d too large", Rk);
    dim3 pg((T_ + DELTA_PREP_TOKENS - 1) / DELTA_PREP_TOKENS, heads);
#define DELTA_SPLIT(TT)                                                                                           \
  do {                                                                                                            \
    B200Q_CUDA(cudaFuncSetAttribute(delta_prepare_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)psm)); \
    delta_prepare_kernel<TT><<<pg, D, psm, st>>>((const TT*)proj, ldp, (const TT*)w2, w0, a_bias, heads, D, Rk, T_, vec); \
    if (D == 32)                                                                                                  \
      delta_recur_kernel<TT, 32><<<sg, 32, 0, st>>>((const TT*)proj, ldp, vec, state, slot_stride, seq_desc, heads, raw); \
    else if (D == 64)                                                                                             \
      delta_recur_kernel<TT, 64><<<sg, 64, 0, st>>>((const TT*)proj, ldp, vec, state, slot_stride, seq_desc, heads, raw); \
    else                                                                                                          \
      delta_recur_kernel<TT, 128><<<sg, 128, 0, st>>>((const TT*)proj, ldp, vec, state, slot_stride, seq_desc, heads, raw); \
    delta_finish_kernel<TT><<<tg, D, 0, st>>>(raw, (const TT*)proj, ldp, out_norm, heads, D, eps, (TT*)out);      \
  } while (0)
    if (dtype == B200Q_DTYPE_F32) DELTA_SPLIT(float);
    else DELTA_SPLIT(bf16);
#undef DELTA_SPLIT
    B200Q_LAUNCH_CHECK();
    return B200Q_OK;
  }
  dim3 grid(n_seqs, heads);
  if (D == 32 || D == 64 || D == 128) {
    const size_t smem = (5 * (size_t)D + (size_t)Rk * (D + 1) + Rk + 32) * sizeof(float);
    B200Q_CHECK_ARG(smem <= 227 * 1024, "delta_rule: decay rank %d does not fit shared memory", Rk);
#define DELTA_REG(TT, DD)                                                                                        \
  do {                                                                                                           \
    B200Q_CUDA(cudaFuncSetAttribute(delta_rule_reg_kernel<TT, DD>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                    (int)smem));                                                                 \
    delta_rule_reg_kernel<TT, DD><<<grid, DD, smem, as_stream(stream)>>>(                                        \
        (const TT*)proj, ldp, (const TT*)w2, w0, a_bias, out_norm, state, slot_stride, seq_desc, heads, Rk, eps, \
        (TT*)out);                                                                                               \
  } while (0)
#define DELTA_BY_D(TT)                    \
  do {                                    \
    if (D == 32) DELTA_REG(TT, 32);       \
    else if (D == 64) DELTA_REG(TT, 64);  \
    else DELTA_REG(TT, 128);              \
  } while (0)
    if (dtype == B200Q_DTYPE_F32) DELTA_BY_D(float);
    else DELTA_BY_D(bf16);
#undef DELTA_BY_D
#undef DELTA_REG
    B200Q_LAUNCH_CHECK();
    return B200Q_OK;
  }
  const int threads = (D + 31) & ~31;
  B200Q_CHECK_ARG(threads <= 1024, "delta_rule: dim=%d unsupported (<= 1024)", D);
  const size_t smem = ((size_t)D * D + 5 * (size_t)D + (size_t)Rk * D + Rk + 32) * sizeof(float);
  B200Q_CHECK_ARG(smem <= 227 * 1024, "delta_rule: a %dx%d state (+ rank %d) does not fit shared memory", D, D, Rk);
  if (dtype == B200Q_DTYPE_F32) {
    B200Q_CUDA(cudaFuncSetAttribute(delta_rule_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    delta_rule_kernel<float><<<grid, threads, smem, as_stream(stream)>>>(
        (const float*)proj, ldp, (const float*)w2, w0, a_bias, out_norm, state, slot_stride, seq_desc, heads, D, Rk,
        eps, (float*)out);
  } else {
    B200Q_CUDA(cudaFuncSetAttribute(delta_rule_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    delta_rule_kernel<bf16><<<grid, threads, smem, as_stream(stream)>>>(
        (const bf16*)proj, ldp, (const bf16*)w2, w0, a_bias, out_norm, state, slot_stride, seq_desc, heads, D, Rk, eps,
        (bf16*)out);
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_polynorm(const void* z, const float* coef, void* y, int rows, int F, float eps, int dtype, void* stream) {
  B200Q_CHECK_ARG(z && coef && y && rows >= 0 && F > 0 && is_dtype(dtype), "polynorm: bad argument");
  if (rows == 0) return B200Q_OK;
  DISPATCH_T(dtype, (polynorm_kernel<T><<<rows, 256, 0, as_stream(stream)>>>((const T*)z, coef, (T*)y, F, eps)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_clamped_glu(const void* gate_up, void* y, int64_t rows, int F, float limit, int dtype, void* stream) {
  B200Q_CHECK_ARG(gate_up && y && rows >= 0 && F > 0 && is_dtype(dtype), "clamped_glu: bad argument");
  if (rows == 0) return B200Q_OK;
  DISPATCH_T(dtype, (clamped_glu_kernel<T><<<grid_for(rows * F), 256, 0, as_stream(stream)>>>((const T*)gate_up, (T*)y,
                                                                                            rows, F, limit)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_moe_route(const float* logits, int T_, int E, int top, int32_t* idx, float* wts, int32_t* group_off,
                    int32_t* perm_tok, int32_t* pair_pos, int32_t* tile_tab, int32_t* n_tiles, void* stream) {
  return b200q_moe_route_ex(logits, T_, E, top, 0, idx, wts, group_off, perm_tok, pair_pos, tile_tab, n_tiles, stream);
}

int b200q_moe_route_ex(const float* logits, int T_, int E, int top, int score_mode, int32_t* idx, float* wts,
                       int32_t* group_off, int32_t* perm_tok, int32_t* pair_pos, int32_t* tile_tab, int32_t* n_tiles,
                       void* stream) {
  B200Q_CHECK_ARG(score_mode == 0 || score_mode == 1, "moe_route: score_mode=%d unknown", score_mode);
  B200Q_CHECK_ARG(!tile_tab == !n_tiles, "moe_route: tile_tab and n_tiles go together");
  B200Q_CHECK_ARG(logits && idx && wts && group_off && perm_tok && pair_pos && T_ >= 0 && E > 0 && top > 0 &&
                      top <= 32 && top <= E && E <= 4096,
                  "moe_route: bad argument (E=%d top=%d)", E, top);
  if (T_ == 0) return B200Q_OK;
  moe_route_kernel<<<(T_ + 3) / 4, 128, 0, as_stream(stream)>>>(logits, T_, E, top, score_mode, idx, wts);
  B200Q_LAUNCH_CHECK();
  moe_plan_kernel<<<1, 1024, (size_t)(3 * E + 1) * sizeof(int32_t), as_stream(stream)>>>(idx, T_ * top, top, E,
                                                                                          group_off, perm_tok, pair_pos,
                                                                                          tile_tab, n_tiles);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_layer_sum(float* x, const void* mix, const void* f, const void* expert_out, const int32_t* pair_pos,
                    const float* wts, int top, const void* shared_out, const float* shared_gate, int T_, int W,
                    int dtype, void* stream) {
  B200Q_CHECK_ARG(x && mix && T_ >= 0 && W > 0 && is_dtype(dtype) && (!expert_out || (pair_pos && wts && top > 0)) &&
                      (!shared_out || shared_gate),
                  "layer_sum: bad argument");
  if (T_ == 0) return B200Q_OK;
  DISPATCH_T(dtype, (layer_sum_kernel<T><<<grid_for((long long)T_ * W), 256, 0, as_stream(stream)>>>(
                        x, (const T*)mix, (const T*)f, (const T*)expert_out, pair_pos, wts, top, (const T*)shared_out,
                        shared_gate, T_, W)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_argmax_f32(const float* logits, int32_t* ids, int B, int V, void* stream) {
  B200Q_CHECK_ARG(logits && ids && B >= 0 && V > 0, "argmax_f32: bad argument");
  if (B == 0) return B200Q_OK;
  argmax_f32_kernel<<<B, 256, 0, as_stream(stream)>>>(logits, ids, V);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_f32_to_bf16(const float* in, void* out, int64_t n, void* stream) {
  B200Q_CHECK_ARG(in && out && n >= 0, "f32_to_bf16: bad argument");
  if (n == 0) return B200Q_OK;
  f32_to_bf16_kernel<<<grid_for(n), 256, 0, as_stream(stream)>>>(in, (bf16*)out, n);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_copy_f32(const float* in, float* out, int64_t n, void* stream) {
  B200Q_CHECK_ARG(in && out && n >= 0, "copy_f32: bad argument");
  if (n == 0) return B200Q_OK;
  copy_f32_kernel<<<grid_for(n), 256, 0, as_stream(stream)>>>(in, out, n);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // extern "C"
