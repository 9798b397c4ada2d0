// window_attn.cu — rotary grouped-query attention over a sliding window.  The paged cache holds, per token, the
// turned keys of every key/value head followed by their values ([kv_heads*dim | kv_heads*vdim], model dtype).
// Rotation pairs dimension i with i + rot_dims/2 over the first rot_dims dimensions of a head (angles and their
// sine / cosine in fp64 from position * freq[i]); the score scale and a per-head temperature are folded into the
// fp32 query; ordinary softmax over the keys max(0, p - window + 1) .. p; one sigmoid gate number per head.
// Options that other designs use: the first `keep_first` keys of a sequence stay visible behind the window (they are
// visited first, as tiles of their own, then the window's keys), and scores may be soft-capped
// (cap * tanh(score / cap)) before the softmax.
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

// step 1 with options: biases, an RMS norm of q and k before rotation (over the whole projection or per head), sine
// and cosine times `mag`, a query temperature that grows with the logarithm of the position, and a layer that writes
// no keys (it reads another layer's cache).  The token's q and k rows are staged in shared memory as fp32.
template <typename T>
__global__ void __launch_bounds__(128) window_attn_prep_opt_kernel(
    const T* __restrict__ proj, int ldp, int q_off, int k_off, int v_off, const float* __restrict__ bias, int heads,
    int kv_heads, int dim, int vdim, int qk_norm, const float* __restrict__ w_qn, const float* __restrict__ w_kn,
    float eps, int rot_dims, const double* __restrict__ freq, float mag, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ slot_mapping, const float* __restrict__ temp, float scale, float temp_coef,
    int temp_every, float* __restrict__ qs, T* __restrict__ cache) {
  extern __shared__ float sh[];
  __shared__ float red[32];
  const int t = blockIdx.x, half = rot_dims / 2, HD = heads * dim, GD = k_off >= 0 ? kv_heads * dim : 0;
  float* cs = sh;                 // [rot_dims/2] cos | [rot_dims/2] sin
  float* qv = sh + rot_dims;      // [heads*dim]
  float* kv = qv + HD;            // [kv_heads*dim]
  const int pos = positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sn, c;
    sincos((double)pos * freq[i], &sn, &c);
    cs[i] = (float)c * mag;
    cs[half + i] = (float)sn * mag;
  }
  const T* pr = proj + (long long)t * ldp;
  for (int e = threadIdx.x; e < HD; e += blockDim.x) qv[e] = ldf(pr + q_off + e) + (bias ? bias[q_off + e] : 0.f);
  for (int e = threadIdx.x; e < GD; e += blockDim.x) kv[e] = ldf(pr + k_off + e) + (bias ? bias[k_off + e] : 0.f);
  __syncthreads();
  if (qk_norm == 1) {  // one norm over all heads of the projection
    for (int which = 0; which < (GD ? 2 : 1); ++which) {
      float* v = which ? kv : qv;
      const float* w = which ? w_kn : w_qn;
      const int n = which ? GD : HD;
      float ss = 0.f;
      for (int e = threadIdx.x; e < n; e += blockDim.x) ss = fmaf(v[e], v[e], ss);
      const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)n + eps);
      for (int e = threadIdx.x; e < n; e += blockDim.x) v[e] = v[e] * inv * w[e];
    }
    __syncthreads();
  } else if (qk_norm == 2) {  // per head, one weight row shared by the heads: warp = head
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int hh = warp; hh < heads + (GD ? kv_heads : 0); hh += nw) {
      float* v = hh < heads ? qv + hh * dim : kv + (hh - heads) * dim;
      const float* w = hh < heads ? w_qn : w_kn;
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) ss = fmaf(v[d], v[d], ss);
      const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dim + eps);
      for (int d = lane; d < dim; d += 32) v[d] = v[d] * inv * w[d];
    }
    __syncthreads();
  }
  auto turned = [&](const float* v, int d) -> float {
    if (d >= rot_dims) return v[d];
    const int i = d < half ? d : d - half;
    const float a = v[i], b = v[i + half];
    return d < half ? a * cs[i] - b * cs[half + i] : b * cs[i] + a * cs[half + i];
  };
  float qmul = scale;
  if (temp_every > 0) qmul *= (float)(1.0 + (double)temp_coef * log((double)((pos + 1) / temp_every) + 1.0));
  for (int e = threadIdx.x; e < HD; e += blockDim.x) {
    const int h = e / dim, d = e % dim;
    qs[(long long)t * HD + e] = turned(qv + h * dim, d) * (qmul * (temp ? temp[h] : 1.f));
  }
  if (k_off < 0) return;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const int GV = kv_heads * vdim;
  T* row = cache + (long long)slot * (GD + GV);
  for (int e = threadIdx.x; e < GD; e += blockDim.x) stf(row + e, turned(kv + (e / dim) * dim, e % dim));
  for (int e = threadIdx.x; e < GV; e += blockDim.x)
    stf(row + GD + e, ldf(pr + v_off + e) + (bias ? bias[v_off + e] : 0.f));
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
                                                          int keep_first, float softcap,
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
  // the kept first keys that the window no longer covers come first (tiles from key 0), then the window's keys
  const int kept = min(keep_first, lo);
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  for (int phase = kept > 0 ? 0 : 1; phase < 2; ++phase)
  for (int j0 = phase ? lo : 0, jend = phase ? p + 1 : kept; j0 < jend; j0 += 32) {
    const int n = min(32, jend - j0);
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
      s = softcap > 0.f ? softcap * tanhf(dot * inv_cap) : dot;
    }
    const float m_new = fmaxf(m, warp_max(s));  // the tile holds at least one visible key: finite
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

// ------------------------------------------------------------------------------------------------
// window attention on the tensor cores (bf16 cache; key and value head sizes of 64 or 128).  One CTA per
// (sequence of the step, key/value head, tile of 16 consecutive tokens of the sequence's portion); warp w serves
// query head w of the group, the 16 tokens are the M rows of mma.sync.m16n8k16 tiles.  Tiles of 64 cached rows
// (keys and values) arrive by cp.async into double-buffered shared memory that all heads of the group read:
// the keys through ldmatrix (S = Q K^T), the values through ldmatrix.trans (O += P V).  Online softmax in fp32
// registers; the weights are rounded to bf16 before they are summed, as the value product sees them.  Key tiles
// start at the first key the tile's first token sees.
// ------------------------------------------------------------------------------------------------
constexpr int WATT_KEYS = 64;
constexpr float WATT_NEG = -1e30f;  // finite floor of the running maximum: exp(masked - floor) = 0, never NaN
template <int D, int DV, bool CAP>
__global__ void __launch_bounds__(256) window_attn_mma_kernel(const float* __restrict__ qs, const bf16* __restrict__ cache,
                                                              const int32_t* __restrict__ block_table, int bt_stride,
                                                              const int32_t* __restrict__ seq_desc, int heads,
                                                              int kv_heads, int block_size, int window,
                                                              int keep_first, float softcap,
                                                              const bf16* __restrict__ gate, int ld_gate,
                                                              bf16* __restrict__ out, int skip_single) {
  constexpr int LDK = D + 8, LDV = DV + 8;  // padded rows (bf16 elements): ldmatrix rows fall on different banks
  extern __shared__ __align__(16) uint8_t smraw[];
  const int nw = blockDim.x >> 5;
  bf16* qsm = reinterpret_cast<bf16*>(smraw);       // [nw][16][LDK]
  bf16* kbuf = qsm + (long long)nw * 16 * LDK;      // [2][64][LDK]
  bf16* vbuf = kbuf + 2 * WATT_KEYS * LDK;          // [2][64][LDV]
  const SeqView sq = seq_view(seq_desc, blockIdx.x);
  const int r0 = blockIdx.z * 16;
  if (r0 >= sq.n || (skip_single && sq.n == 1)) return;  // single tokens: the decode kernel's
  const int nrows = min(16, sq.n - r0);
  const int rep = heads / kv_heads, parts = (rep + nw - 1) / nw;
  const int g = blockIdx.y / parts, part = blockIdx.y % parts;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, q4 = lane & 3;
  const int hg = part * nw + warp;
  const bool live = hg < rep;
  const int h = g * rep + (live ? hg : 0);
  const int p_first = sq.pos0 + r0, p_last = p_first + nrows - 1;
  const int lo_first = window > 0 ? max(0, p_first - window + 1) : 0;
  const int32_t* bt = block_table + (long long)blockIdx.x * bt_stride;
  const int GD = kv_heads * D, RS = GD + kv_heads * DV;
  // kept first keys that the first token's window no longer covers: whole tiles from key 0, before the window's
  const int kept = min(keep_first, lo_first), nst = (kept + WATT_KEYS - 1) / WATT_KEYS;
  const int ntiles = nst + (p_last - lo_first) / WATT_KEYS + 1;
  auto tile_start = [&](int c) { return c < nst ? c * WATT_KEYS : lo_first + (c - nst) * WATT_KEYS; };
  const float inv_cap = CAP ? 1.f / softcap : 0.f;

  auto load_tile = [&](int c, int buf) {
    const int j0 = tile_start(c);
    bf16* kb = kbuf + (long long)buf * WATT_KEYS * LDK;
    bf16* vb = vbuf + (long long)buf * WATT_KEYS * LDV;
    constexpr int CK = D / 8, CV = DV / 8, CPR = CK + CV;  // 16-byte pieces of a cached row's key and value
    for (int e = tid; e < WATT_KEYS * CPR; e += blockDim.x) {
      const int j = e / CPR, ck = e % CPR, pos = j0 + j;
      bf16* dst = ck < CK ? kb + j * LDK + ck * 8 : vb + j * LDV + (ck - CK) * 8;
      if (pos <= p_last) {
        const long long row = (long long)bt[pos / block_size] * block_size + pos % block_size;
        const bf16* src = ck < CK ? cache + row * RS + (long long)g * D + ck * 8
                                  : cache + row * RS + GD + (long long)g * DV + (ck - CK) * 8;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load_tile(0, 0);
  // the queries of this CTA's heads (scale and temperature folded in), bf16, rows past the portion are zeros
  for (int e = tid; e < nw * 16 * D; e += blockDim.x) {
    const int w = e / (16 * D), r = (e / D) % 16, d = e % D, hh = part * nw + w;
    const float v = (hh < rep && r < nrows) ? qs[((long long)(sq.row0 + r0 + r) * heads + g * rep + hh) * D + d] : 0.f;
    qsm[((long long)w * 16 + r) * LDK + d] = __float2bfloat16_rn(v);
  }
  const uint32_t q_s = smem_u32(qsm + (long long)warp * 16 * LDK);
  const uint32_t a_off = (uint32_t)(((lane & 15) * LDK + (lane >> 4) * 8) * 2);
  const uint32_t kq_off = (uint32_t)((((lane & 7) + 8 * (lane >> 4)) * LDK + 8 * ((lane >> 3) & 1)) * 2);
  // rows gq and gq + 8 of the tile belong to this thread
  int p_row[2], lo_row[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = gq + 8 * r;
    p_row[r] = i < nrows ? p_first + i : -1;  // a dead row sees no key
    lo_row[r] = (window > 0 && i < nrows) ? max(0, p_row[r] - window + 1) : 0;
  }
  float m_[2] = {WATT_NEG, WATT_NEG}, l_[2] = {0.f, 0.f};
  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int c = 0; c < ntiles; ++c) {
    const int buf = c & 1, j0 = tile_start(c);
    const bool sink_tile = c < nst;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // tile c (and, first time, the queries) is in shared memory; tile c-1 is done with
    if (c + 1 < ntiles) load_tile(c + 1, buf ^ 1);
    if (!live) continue;
    const uint32_t kb_s = smem_u32(kbuf + (long long)buf * WATT_KEYS * LDK);
    const uint32_t vb_s = smem_u32(vbuf + (long long)buf * WATT_KEYS * LDV);
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(q_s + a_off + ks * 32, a0, a1, a2, a3);
#pragma unroll
      for (int nt2 = 0; nt2 < 4; ++nt2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kb_s + kq_off + (uint32_t)(nt2 * 16 * LDK * 2 + ks * 32), b0, b1, b2, b3);
        mma_bf16_16816(s[2 * nt2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(s[2 * nt2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    float rmax[2] = {WATT_NEG, WATT_NEG};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + nt * 8 + 2 * q4 + (e & 1), r = e >> 1;
        const bool see = sink_tile ? (j < kept && p_row[r] >= 0) : (j <= p_row[r] && (j >= lo_row[r] || j < keep_first));
        const float sc = CAP ? softcap * tanhf(s[nt][e] * inv_cap) : s[nt][e];
        const float v = see ? sc : -INFINITY;
        s[nt][e] = v;
        rmax[r] = fmaxf(rmax[r], v);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 1));
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 2));
      const float mn = fmaxf(m_[r], rmax[r]);
      corr[r] = __expf(m_[r] - mn);
      m_[r] = mn;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = round_bf16(__expf(s[nt][e] - m_[e >> 1]));  // masked: exp(-inf) = 0
        s[nt][e] = pv;
        psum[e >> 1] += pv;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_[r] = l_[r] * corr[r] + psum[r];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
#pragma unroll
    for (int kk2 = 0; kk2 < WATT_KEYS / 16; ++kk2) {
      const uint32_t a0 = pack_bf16x2(s[2 * kk2][0], s[2 * kk2][1]), a1 = pack_bf16x2(s[2 * kk2][2], s[2 * kk2][3]);
      const uint32_t a2 = pack_bf16x2(s[2 * kk2 + 1][0], s[2 * kk2 + 1][1]),
                     a3 = pack_bf16x2(s[2 * kk2 + 1][2], s[2 * kk2 + 1][3]);
      const int key = kk2 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const uint32_t v_row = vb_s + (uint32_t)((key * LDV + 8 * (lane >> 4)) * 2);
#pragma unroll
      for (int nd2 = 0; nd2 < DV / 16; ++nd2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(v_row + nd2 * 32, b0, b1, b2, b3);
        mma_bf16_16816(o[2 * nd2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(o[2 * nd2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  if (!live) return;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_[r] += __shfl_xor_sync(0xffffffffu, l_[r], 1);
    l_[r] += __shfl_xor_sync(0xffffffffu, l_[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = gq + 8 * r;
    if (i >= nrows) continue;
    const long long t = sq.row0 + r0 + i;
    const float gv = gate ? sigmoidf_(__bfloat162float(gate[t * ld_gate + h])) : 1.f;
    const float inv = gv / l_[r];
    bf16* orow = out + (t * heads + h) * DV;
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt) {
      const int d = nt * 8 + 2 * q4;
      *reinterpret_cast<uint32_t*>(orow + d) = pack_bf16x2(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// The same for a single decoded token of a sequence: one CTA (4 warps) per (sequence, key/value head).  The M
// rows of the tiles are the query heads of the group (<= 16), so one pass over the cached rows serves all of
// them; warp w takes the key tiles w, w+4, ... (16 or 32 cached rows each) of the token's window through its own
// double-buffered cp.async ring (no CTA barrier inside the loop) and keeps its own softmax state; the four states
// are merged through shared memory in a fixed order at the end.  The tile size is chosen so that three CTAs fit
// an SM: the kernel lives on loads in flight, not on arithmetic.
// ------------------------------------------------------------------------------------------------
constexpr int WDEC_WARPS = 4;
template <int D, int DV, int WDEC_KEYS, bool CAP>
__global__ void __launch_bounds__(128) window_attn_decode_mma_kernel(const float* __restrict__ qs,
                                                                     const bf16* __restrict__ cache,
                                                                     const int32_t* __restrict__ block_table,
                                                                     int bt_stride, const int32_t* __restrict__ seq_desc,
                                                                     int heads, int kv_heads, int block_size, int window,
                                                                     int keep_first, float softcap,
                                                                     const bf16* __restrict__ gate, int ld_gate,
                                                                     bf16* __restrict__ out) {
  constexpr int LDK = D + 8, LDV = DV + 8, MS = DV + 2;
  extern __shared__ __align__(16) uint8_t smraw[];
  bf16* qsm = reinterpret_cast<bf16*>(smraw);    // [16][LDK]
  bf16* kvbuf = qsm + 16 * LDK;                  // [4 warps][2][32][LDK + LDV]
  float* mrg = reinterpret_cast<float*>(kvbuf);  // after the loop: [4][16][DV + 2]
  const SeqView sq = seq_view(seq_desc, blockIdx.x);
  if (sq.n != 1) return;  // portions of prompts take the tile kernel
  const int g = blockIdx.y, rep = heads / kv_heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, q4 = lane & 3;
  const int p = sq.pos0, lo = window > 0 ? max(0, p - window + 1) : 0;
  const long long t = sq.row0;
  const int32_t* bt = block_table + (long long)blockIdx.x * bt_stride;
  const int GD = kv_heads * D, RS = GD + kv_heads * DV;
  const int kept = min(keep_first, lo), nst = (kept + WDEC_KEYS - 1) / WDEC_KEYS;  // kept first keys: tiles of their own
  const int ntiles = nst + (p - lo) / WDEC_KEYS + 1;
  auto tile_start = [&](int c) { return c < nst ? c * WDEC_KEYS : lo + (c - nst) * WDEC_KEYS; };
  const float inv_cap = CAP ? 1.f / softcap : 0.f;
  bf16* kw = kvbuf + (long long)warp * 2 * WDEC_KEYS * (LDK + LDV);

  auto load_tile = [&](int c, int buf) {  // by this warp alone
    const int j0 = tile_start(c);
    bf16* kb = kw + (long long)buf * WDEC_KEYS * (LDK + LDV);
    bf16* vb = kb + WDEC_KEYS * LDK;
    constexpr int CK = D / 8, CV = DV / 8, CPR = CK + CV;
    for (int e = lane; e < WDEC_KEYS * CPR; e += 32) {
      const int j = e / CPR, ck = e % CPR, pos = j0 + j;
      bf16* dst = ck < CK ? kb + j * LDK + ck * 8 : vb + j * LDV + (ck - CK) * 8;
      if (pos <= p) {
        const long long row = (long long)bt[pos / block_size] * block_size + pos % block_size;
        const bf16* src = ck < CK ? cache + row * RS + (long long)g * D + ck * 8
                                  : cache + row * RS + GD + (long long)g * DV + (ck - CK) * 8;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (warp < ntiles) load_tile(warp, 0);
  for (int e = tid; e < 16 * D; e += blockDim.x) {
    const int r = e / D, d = e % D;
    qsm[r * LDK + d] = __float2bfloat16_rn(r < rep ? qs[(t * heads + g * rep + r) * D + d] : 0.f);
  }
  __syncthreads();
  const uint32_t q_s = smem_u32(qsm);
  const uint32_t a_off = (uint32_t)(((lane & 15) * LDK + (lane >> 4) * 8) * 2);
  const uint32_t kq_off = (uint32_t)((((lane & 7) + 8 * (lane >> 4)) * LDK + 8 * ((lane >> 3) & 1)) * 2);
  const bool row_on[2] = {gq < rep, gq + 8 < rep};
  float m_[2] = {WATT_NEG, WATT_NEG}, l_[2] = {0.f, 0.f};
  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int c = warp, it = 0; c < ntiles; c += WDEC_WARPS, ++it) {
    const int buf = it & 1, j0 = tile_start(c), jend = c < nst ? kept : p + 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    if (c + WDEC_WARPS < ntiles) load_tile(c + WDEC_WARPS, buf ^ 1);
    const bf16* kb = kw + (long long)buf * WDEC_KEYS * (LDK + LDV);
    const uint32_t kb_s = smem_u32(kb), vb_s = smem_u32(kb + WDEC_KEYS * LDK);
    constexpr int NT = WDEC_KEYS / 8;  // 8-key score tiles of a key tile
    float s[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(q_s + a_off + ks * 32, a0, a1, a2, a3);
#pragma unroll
      for (int nt2 = 0; nt2 < NT / 2; ++nt2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kb_s + kq_off + (uint32_t)(nt2 * 16 * LDK * 2 + ks * 32), b0, b1, b2, b3);
        mma_bf16_16816(s[2 * nt2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(s[2 * nt2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    float rmax[2] = {WATT_NEG, WATT_NEG};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + nt * 8 + 2 * q4 + (e & 1), r = e >> 1;
        const float sc = CAP ? softcap * tanhf(s[nt][e] * inv_cap) : s[nt][e];
        const float v = (row_on[r] && j < jend) ? sc : -INFINITY;  // tiles start at the window's first key
        s[nt][e] = v;
        rmax[r] = fmaxf(rmax[r], v);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 1));
      rmax[r] = fmaxf(rmax[r], __shfl_xor_sync(0xffffffffu, rmax[r], 2));
      const float mn = fmaxf(m_[r], rmax[r]);
      corr[r] = __expf(m_[r] - mn);
      m_[r] = mn;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = round_bf16(__expf(s[nt][e] - m_[e >> 1]));
        s[nt][e] = pv;
        psum[e >> 1] += pv;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_[r] = l_[r] * corr[r] + psum[r];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
#pragma unroll
    for (int kk2 = 0; kk2 < WDEC_KEYS / 16; ++kk2) {
      const uint32_t a0 = pack_bf16x2(s[2 * kk2][0], s[2 * kk2][1]), a1 = pack_bf16x2(s[2 * kk2][2], s[2 * kk2][3]);
      const uint32_t a2 = pack_bf16x2(s[2 * kk2 + 1][0], s[2 * kk2 + 1][1]),
                     a3 = pack_bf16x2(s[2 * kk2 + 1][2], s[2 * kk2 + 1][3]);
      const int key = kk2 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const uint32_t v_row = vb_s + (uint32_t)((key * LDV + 8 * (lane >> 4)) * 2);
#pragma unroll
      for (int nd2 = 0; nd2 < DV / 16; ++nd2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(v_row + nd2 * 32, b0, b1, b2, b3);
        mma_bf16_16816(o[2 * nd2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(o[2 * nd2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  // ---- merge the four warps' states: [warp][row][DV + 2] = (o..., m, l); a warp without tiles holds (0, floor, 0) ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_[r] += __shfl_xor_sync(0xffffffffu, l_[r], 1);
    l_[r] += __shfl_xor_sync(0xffffffffu, l_[r], 2);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();  // every warp is done with its buffers: they become the merge area
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float* dst = mrg + ((long long)warp * 16 + gq + 8 * r) * MS;
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt) {
      dst[nt * 8 + 2 * q4] = o[nt][2 * r];
      dst[nt * 8 + 2 * q4 + 1] = o[nt][2 * r + 1];
    }
    if (q4 == 0) {
      dst[DV] = m_[r];
      dst[DV + 1] = l_[r];
    }
  }
  __syncthreads();
  for (int e = tid; e < rep * DV; e += blockDim.x) {
    const int r = e / DV, d = e % DV;
    float mx = WATT_NEG;
#pragma unroll
    for (int w = 0; w < WDEC_WARPS; ++w) mx = fmaxf(mx, mrg[((long long)w * 16 + r) * MS + DV]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < WDEC_WARPS; ++w) {
      const float* src = mrg + ((long long)w * 16 + r) * MS;
      const float f = expf(src[DV] - mx);
      num = fmaf(src[d], f, num);
      den = fmaf(src[DV + 1], f, den);
    }
    const int h = g * rep + r;
    const float gv = gate ? sigmoidf_(__bfloat162float(gate[t * ld_gate + h])) : 1.f;
    out[(t * heads + h) * DV + d] = __float2bfloat16_rn(num / den * gv);
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

int b200q_window_attn_prep_ex(const void* proj, int ldp, int q_off, int k_off, int v_off, const float* bias, int heads,
                              int kv_heads, int dim, int vdim, int qk_norm, const float* w_qn, const float* w_kn, float eps,
                              int rot_dims, const double* freq, float mag, const int32_t* positions,
                              const int32_t* slot_mapping, const float* temp, float scale, float temp_coef, int temp_every,
                              float* qs, void* cache, int T_, int dtype, void* stream) {
  const bool own = k_off >= 0;
  B200Q_CHECK_ARG(proj && positions && qs && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && q_off >= 0 &&
                      ldp >= q_off + heads * dim && rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim &&
                      (rot_dims == 0 || freq) && T_ >= 0 && is_dtype(dtype) && temp_every >= 0,
                  "window_attn_prep: bad argument (heads=%d kv_heads=%d dim=%d vdim=%d rot_dims=%d even, <= dim)", heads,
                  kv_heads, dim, vdim, rot_dims);
  B200Q_CHECK_ARG(!own || (slot_mapping && cache && v_off >= 0 && ldp >= k_off + kv_heads * dim &&
                           ldp >= v_off + kv_heads * vdim),
                  "window_attn_prep: bad key / value columns (k_off=%d v_off=%d ldp=%d)", k_off, v_off, ldp);
  B200Q_CHECK_ARG(qk_norm >= 0 && qk_norm <= 2 && (qk_norm == 0 || (w_qn && (!own || w_kn))) && eps >= 0.f,
                  "window_attn_prep: bad query / key norm (%d)", qk_norm);
  if (T_ == 0) return B200Q_OK;
  const size_t smem = (size_t)(std::max(rot_dims, 1) + heads * dim + kv_heads * dim) * sizeof(float);
  B200Q_CHECK_ARG(smem <= 200 * 1024, "window_attn_prep: heads * dim too large for one CTA");
  DISPATCH_T(dtype, {
    auto kern = window_attn_prep_opt_kernel<T>;
    if (smem > 48 * 1024) B200Q_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<T_, 128, smem, as_stream(stream)>>>((const T*)proj, ldp, q_off, k_off, v_off, bias, heads, kv_heads, dim, vdim,
                                               qk_norm, w_qn, w_kn, eps, rot_dims, freq, mag, positions, slot_mapping,
                                               temp, scale, temp_coef, temp_every, qs, (T*)cache);
  });
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

static int window_attn_mma_mode() {  // B200Q_WINDOW_ATTN_MMA=0: the scalar kernel everywhere
  static const int mode = [] {
    const char* v = getenv("B200Q_WINDOW_ATTN_MMA");
    return v ? atoi(v) : 1;
  }();
  return mode;
}

// cached rows per tile of the decode kernel: 32, or 16 where 32 would leave room for one CTA per SM only
// (B200Q_WINDOW_DECODE_KEYS = 16 / 32 overrides)
static int window_attn_decode_keys(int dim, int vdim) {
  static const int forced = [] {
    const char* v = getenv("B200Q_WINDOW_DECODE_KEYS");
    return v ? atoi(v) : 0;
  }();
  if (forced == 16 || forced == 32) return forced;
  return dim + vdim > 128 ? 16 : 32;
}

int b200q_window_attn(const float* qs, const void* cache, const int32_t* block_table, int bt_stride, const int32_t* row_seq,
                      const int32_t* positions, const int32_t* seq_desc, int n_seqs, int T_, int heads, int kv_heads,
                      int dim, int vdim, int block_size, int window, const void* gate, int ld_gate, void* out, int dtype,
                      void* stream) {
  return b200q_window_attn_ex(qs, cache, block_table, bt_stride, row_seq, positions, seq_desc, n_seqs, T_, heads, kv_heads,
                              dim, vdim, block_size, window, 0, 0.f, gate, ld_gate, out, dtype, stream);
}

int b200q_window_attn_ex(const float* qs, const void* cache, const int32_t* block_table, int bt_stride,
                         const int32_t* row_seq, const int32_t* positions, const int32_t* seq_desc, int n_seqs, int T_,
                         int heads, int kv_heads, int dim, int vdim, int block_size, int window, int keep_first,
                         float softcap, const void* gate, int ld_gate, void* out, int dtype, void* stream) {
  B200Q_CHECK_ARG(keep_first >= 0 && softcap >= 0.f, "window_attn: bad kept keys (%d) or soft cap (%g)", keep_first,
                  (double)softcap);
  if (window <= 0) keep_first = 0;  // every earlier key is visible anyway
  B200Q_CHECK_ARG(qs && cache && block_table && row_seq && positions && out && heads > 0 && kv_heads > 0 &&
                      heads % kv_heads == 0 && dim > 0 && dim <= 512 && vdim > 0 && vdim <= 512 && block_size > 0 &&
                      window >= 0 && T_ >= 0 && is_dtype(dtype) && (!gate || ld_gate >= heads),
                  "window_attn: bad argument (heads=%d kv_heads=%d dim=%d vdim=%d, both <= 512)", heads, kv_heads, dim,
                  vdim);
  if (T_ == 0) return B200Q_OK;
  cudaStream_t st = as_stream(stream);
  const int rep = heads / kv_heads;
  // bf16 caches with head sizes the tensor-core tiles take, when the caller gives the per-sequence view
  if (seq_desc && n_seqs > 0 && dtype == B200Q_DTYPE_BF16 && (dim == 64 || dim == 128) && (vdim == 64 || vdim == 128) &&
      window_attn_mma_mode() && ((reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    const int nw = rep < 8 ? rep : 8, parts = (rep + nw - 1) / nw;
    const int ztiles = (T_ - n_seqs + 1 + 15) / 16;  // no portion of this step is longer than T - (n_seqs - 1)
    dim3 mgrid(n_seqs, kv_heads * parts, ztiles);
    B200Q_CHECK_ARG(mgrid.y <= 65535 && mgrid.z <= 65535, "window_attn: step too large (%d tokens)", T_);
    const size_t msm = ((size_t)nw * 16 + 2 * WATT_KEYS) * (dim + 8) * 2 + (size_t)2 * WATT_KEYS * (vdim + 8) * 2;
    // single decoded tokens go to the kernel whose rows are the heads of a group (groups of up to 16 heads); a
    // step of single tokens only (T == n_seqs) needs no tile kernel
    const bool dec = rep <= 16, tiles = !dec || T_ > n_seqs;
    const int dkeys = window_attn_decode_keys(dim, vdim);
    const size_t dsm = std::max((size_t)16 * (dim + 8) * 2 + (size_t)WDEC_WARPS * 2 * dkeys * (dim + vdim + 16) * 2,
                                (size_t)16 * (dim + 8) * 2 + (size_t)WDEC_WARPS * 16 * (vdim + 2) * 4);
    dim3 dgrid(n_seqs, kv_heads);
#define MMA_ATTN(DD, DDV)                                                                                                \
  do {                                                                                                                   \
    if (softcap > 0.f) MMA_ATTN_C(DD, DDV, true);                                                                        \
    else MMA_ATTN_C(DD, DDV, false);                                                                                     \
  } while (0)
#define MMA_ATTN_C(DD, DDV, CC)                                                                                              \
  do {                                                                                                                   \
    if (tiles) {                                                                                                         \
      if (msm > 48 * 1024)                                                                                               \
        B200Q_CUDA(cudaFuncSetAttribute(window_attn_mma_kernel<DD, DDV, CC>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                        (int)msm));                                                                      \
      window_attn_mma_kernel<DD, DDV, CC><<<mgrid, nw * 32, msm, st>>>(qs, (const bf16*)cache, block_table, bt_stride,       \
                                                                   seq_desc, heads, kv_heads, block_size, window,        \
                                                                   keep_first, softcap,                                  \
                                                                   (const bf16*)gate, ld_gate, (bf16*)out, dec ? 1 : 0); \
      B200Q_LAUNCH_CHECK();                                                                                              \
    }                                                                                                                    \
    if (dec) {                                                                                                           \
      auto dk = dkeys == 16 ? window_attn_decode_mma_kernel<DD, DDV, 16, CC> : window_attn_decode_mma_kernel<DD, DDV, 32, CC>;   \
      if (dsm > 48 * 1024)                                                                                               \
        B200Q_CUDA(cudaFuncSetAttribute(dk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsm));                     \
      dk<<<dgrid, 128, dsm, st>>>(qs, (const bf16*)cache, block_table, bt_stride, seq_desc, heads, kv_heads, block_size, \
                                  window, keep_first, softcap, (const bf16*)gate, ld_gate, (bf16*)out);                  \
      B200Q_LAUNCH_CHECK();                                                                                              \
    }                                                                                                                    \
  } while (0)
    if (dim == 64 && vdim == 64) MMA_ATTN(64, 64);
    else if (dim == 64) MMA_ATTN(64, 128);
    else if (vdim == 64) MMA_ATTN(128, 64);
    else MMA_ATTN(128, 128);
#undef MMA_ATTN
#undef MMA_ATTN_C
    return B200Q_OK;
  }
  dim3 grid(T_, kv_heads, (rep + 7) / 8);
  B200Q_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "window_attn: too many heads");
  const size_t smem = (size_t)(8 * dim + 32 * (dim + 1) + 32 * (vdim + 1)) * sizeof(float);
#define SCALAR(ACC)                                                                                                       \
  do {                                                                                                                    \
    DISPATCH_T(dtype, {                                                                                                   \
      auto kern = window_attn_kernel<T, ACC>;                                                                             \
      if (smem > 48 * 1024) B200Q_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      kern<<<grid, 256, smem, st>>>(qs, (const T*)cache, block_table, bt_stride, row_seq, positions, heads, kv_heads, dim, \
                                    vdim, block_size, window, keep_first, softcap, (const T*)gate, ld_gate, (T*)out);      \
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
