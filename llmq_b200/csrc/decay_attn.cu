// decay_attn.cu — linear attention with decay: per (sequence, head) an fp32 state S [dim][vdim] that is
// multiplied by a decay and receives the outer product k v^T at every token.  Two forms share one kernel:
//   constant decay per head:          S <- decay_h S + k v^T;   o = S^T q                        (reads the new state)
//   decay per token and key channel:  o = (S + diag(bonus) k v^T)^T q;   S <- diag(w) S + k v^T  (reads the old one)
// followed by a norm over groups of the output row, a weight and a gate (gated_rmsnorm_kernel).
//
// One warp per (sequence, head, 8 or 16 value columns): columns of the state are independent, so a head spreads
// over many CTAs; four lanes share a column, each with a quarter of it (zero-padded) in
// registers, partial dot products summed by butterfly shuffles.  q, k (and w) of 8 tokens at a time arrive
// in shared memory by cp.async one group ahead, v of the group is prefetched into registers.  The order of
// every sum is fixed, so a token's output does not depend on how the prompt was cut.
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

constexpr int DATT_G = 8;  // tokens staged per group
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

// VECW: decay per token and key channel (with the bonus); else one constant per head.  NC: value columns per lane
// group (the warp covers 8 * NC columns): with two, every k / q / w vector read from shared memory serves twice
// as many multiply-adds and each lane carries two independent chains.
// LPC: lanes that share a column (the warp covers 32 / LPC * NC columns).
template <int DT, bool VECW, int NC, int LPC>
__global__ void __launch_bounds__(32) decay_attn_kernel(const float* __restrict__ qkv, int ldq, int q_off, int k_off,
                                                        int v_off, const float* __restrict__ head_decay,
                                                        const float* __restrict__ w, int ldw,
                                                        const float* __restrict__ bonus, float* __restrict__ state,
                                                        long long slot_stride, const int32_t* __restrict__ seq_desc,
                                                        int heads, int dim, int vdim, float* __restrict__ raw) {
  constexpr int QL = DT / LPC;         // state values per lane and column
  constexpr int CW = 32 / LPC;         // columns of a warp per NC
  constexpr int NV = VECW ? 3 : 2;     // vectors per token in shared memory: k, q (, w)
  extern __shared__ __align__(16) float sm[];  // [2][G][NV*DT]
  const SeqView s = seq_view(seq_desc, blockIdx.x);
  if (s.n <= 0) return;
  const int h = blockIdx.y, lane = threadIdx.x, sub = lane / CW, j0 = blockIdx.z * (CW * NC) + lane % CW;
  const int q0 = sub * QL, HV = heads * vdim;
  bool on[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) on[c] = j0 + CW * c < vdim;
  const bool vec = (dim & 3) == 0 && (ldq & 3) == 0 && (q_off & 3) == 0 && (k_off & 3) == 0 &&
                   (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 &&
                   (!VECW || ((ldw & 3) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0));
  float* st = state + (long long)s.slot * slot_stride + (long long)h * dim * vdim;
  for (int e = lane; e < 2 * DATT_G * NV * DT; e += 32) sm[e] = 0.f;  // the padding stays zero
  __syncwarp();
  const float* krow = qkv + k_off + h * dim;
  const float* qrow = qkv + q_off + h * dim;
  const float* wrow = VECW ? w + h * dim : nullptr;
  // the 16-byte pieces of a token's vectors that this lane copies are the same for every token: where each comes
  // from and where it lands is worked out once, so that a group's copies cost no index arithmetic
  constexpr int NP = (NV * DT / 4 + 31) / 32;
  const float* psrc[NP];
  long long pld[NP];
  int pdst[NP];
  {
    const int pv = dim / 4, per = NV * pv;
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      const int pc = lane + 32 * i, which = pc / max(pv, 1), off = (pc - which * pv) * 4;
      const bool live = vec && pc < per;
      psrc[i] = !live ? nullptr : (which == 0 ? krow : which == 1 ? qrow : wrow) + off;
      pld[i] = which == 2 ? ldw : ldq;
      pdst[i] = which * DT + off;
    }
  }
  auto fetch = [&](int g0, int buf) {
    const int cnt = min(DATT_G, s.n - g0);
    float* dst0 = sm + (long long)buf * DATT_G * NV * DT;
    if (vec) {
      const long long row = s.row0 + g0;
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        if (!psrc[i]) continue;
        const float* src = psrc[i] + row * pld[i];
        float* dst = dst0 + pdst[i];
        for (int tk = 0; tk < cnt; ++tk, src += pld[i], dst += NV * DT) cp_async16(dst, src);
      }
    } else {
      for (int e = lane; e < cnt * NV * dim; e += 32) {
        const int tk = e / (NV * dim), i = e % (NV * dim), which = i / dim, d = i % dim;
        const long long row = s.row0 + g0 + tk;
        dst0[tk * NV * DT + which * DT + d] =
            which == 0 ? krow[row * ldq + d] : which == 1 ? qrow[row * ldq + d] : wrow[row * ldw + d];
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(0, 0);
  float S[NC][QL], U[VECW ? QL : 1];
#pragma unroll
  for (int c = 0; c < NC; ++c)
#pragma unroll
    for (int q = 0; q < QL; ++q)
      S[c][q] = (on[c] && q0 + q < dim && s.pos0 > 0) ? st[(long long)(q0 + q) * vdim + j0 + CW * c] : 0.f;
  if (VECW) {
#pragma unroll
    for (int q = 0; q < QL; ++q) U[q] = q0 + q < dim ? bonus[h * dim + q0 + q] : 0.f;
  }
  const float lam = VECW ? 1.f : head_decay[h];
  const float* vcol = qkv + v_off + h * vdim + j0;
  float* rcol = raw + h * vdim + j0;
  for (int g0 = 0, buf = 0; g0 < s.n; g0 += DATT_G, buf ^= 1) {
    const int cnt = min(DATT_G, s.n - g0);
    float vj[NC][DATT_G];
    const float* vrow = vcol + (long long)(s.row0 + g0) * ldq;
    float* rrow = rcol + (long long)(s.row0 + g0) * HV;
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
      for (int tk = 0; tk < DATT_G; ++tk) vj[c][tk] = (on[c] && tk < cnt) ? vrow[(long long)tk * ldq + CW * c] : 0.f;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();  // this group has landed; the other buffer is no longer read
    if (g0 + DATT_G < s.n) fetch(g0 + DATT_G, buf ^ 1);
    const float* base = sm + (long long)buf * DATT_G * NV * DT + q0;
#pragma unroll
    for (int tk = 0; tk < DATT_G; ++tk) {
      if (tk < cnt) {
        const float4* k4 = reinterpret_cast<const float4*>(base + tk * NV * DT);
        const float4* q4 = reinterpret_cast<const float4*>(base + tk * NV * DT + DT);
        const float4* w4 = reinterpret_cast<const float4*>(base + tk * NV * DT + (VECW ? 2 * DT : 0));
        float o[NC][4];
#pragma unroll
        for (int c = 0; c < NC; ++c) o[c][0] = o[c][1] = o[c][2] = o[c][3] = 0.f;
#pragma unroll
        for (int q = 0; q < QL / 4; ++q) {
          const float4 k = k4[q], qq = q4[q];
          float4 ww;
          if (VECW) ww = w4[q];
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            const float v = vj[c][tk];
            float* Sc = S[c] + 4 * q;
            if (VECW) {
              const float a0 = k.x * v, a1 = k.y * v, a2 = k.z * v, a3 = k.w * v;
              o[c][0] = fmaf(fmaf(U[4 * q], a0, Sc[0]), qq.x, o[c][0]);
              o[c][1] = fmaf(fmaf(U[4 * q + 1], a1, Sc[1]), qq.y, o[c][1]);
              o[c][2] = fmaf(fmaf(U[4 * q + 2], a2, Sc[2]), qq.z, o[c][2]);
              o[c][3] = fmaf(fmaf(U[4 * q + 3], a3, Sc[3]), qq.w, o[c][3]);
              Sc[0] = fmaf(ww.x, Sc[0], a0);
              Sc[1] = fmaf(ww.y, Sc[1], a1);
              Sc[2] = fmaf(ww.z, Sc[2], a2);
              Sc[3] = fmaf(ww.w, Sc[3], a3);
            } else {
              Sc[0] = fmaf(lam, Sc[0], k.x * v);
              Sc[1] = fmaf(lam, Sc[1], k.y * v);
              Sc[2] = fmaf(lam, Sc[2], k.z * v);
              Sc[3] = fmaf(lam, Sc[3], k.w * v);
              o[c][0] = fmaf(Sc[0], qq.x, o[c][0]);
              o[c][1] = fmaf(Sc[1], qq.y, o[c][1]);
              o[c][2] = fmaf(Sc[2], qq.z, o[c][2]);
              o[c][3] = fmaf(Sc[3], qq.w, o[c][3]);
            }
          }
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          float t = (o[c][0] + o[c][1]) + (o[c][2] + o[c][3]);
#pragma unroll
          for (int off = CW; off < 32; off <<= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
          if (on[c] && sub == 0) rrow[(long long)tk * HV + CW * c] = t;
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < NC; ++c)
    if (on[c]) {
#pragma unroll
      for (int q = 0; q < QL; ++q)
        if (q0 + q < dim) st[(long long)(q0 + q) * vdim + j0 + CW * c] = S[c][q];
    }
}

// out = raw / rms(group) * w * act(gate): CTA per (token, group of `group` consecutive values)
template <typename T>
__global__ void __launch_bounds__(256) gated_rmsnorm_kernel(const float* __restrict__ raw, int C, int group,
                                                            const float* __restrict__ w, const T* __restrict__ gate,
                                                            int ld_gate, int gate_act, float eps, T* __restrict__ out) {
  __shared__ float red[32];
  const int t = blockIdx.x, c0 = blockIdx.y * group;
  const float* r = raw + (long long)t * C + c0;
  float ss = 0.f;
  for (int c = threadIdx.x; c < group; c += blockDim.x) ss = fmaf(r[c], r[c], ss);
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)group + eps);
  const T* g = gate + (long long)t * ld_gate + c0;
  T* o = out + (long long)t * C + c0;
  for (int c = threadIdx.x; c < group; c += blockDim.x) {
    const float gv = ldf(g + c);
    stf(o + c, r[c] * inv * w[c0 + c] * (gate_act == 1 ? siluf_(gv) : sigmoidf_(gv)));
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_decay_attn(const float* qkv, int ldq, int q_off, int k_off, int v_off, const float* head_decay,
                     const float* w, int ldw, const float* bonus, float* state, long long slot_stride,
                     const int32_t* seq_desc, int n_seqs, int heads, int dim, int vdim, float* raw, void* stream) {
  B200Q_CHECK_ARG(qkv && state && seq_desc && raw && heads > 0 && dim > 0 && dim <= 256 && vdim > 0 && n_seqs >= 0 &&
                      q_off >= 0 && k_off >= 0 && v_off >= 0,
                  "decay_attn: bad argument (heads=%d dim=%d (<= 256) vdim=%d)", heads, dim, vdim);
  B200Q_CHECK_ARG((head_decay != nullptr) != (w != nullptr) && (!w || (bonus && ldw >= heads * dim)),
                  "decay_attn: give either a decay per head, or a decay per token and channel with its bonus");
  if (n_seqs == 0) return B200Q_OK;
  cudaStream_t st = as_stream(stream);
  // Many (sequence, head) pairs (decode) take two value columns per lane group while the state fits the registers
  // (key sizes up to 64); few pairs (prompts) keep one, which gives twice the warps.  A column's sums have the
  // same order in both, so the choice changes no result.  (Eight lanes per column were tried for prompt steps:
  // no gain, a warp's time per token is its dependent instruction chain, not its multiply-adds.)
  static const int forced = [] {  // B200Q_DECAY_ATTN_SPLIT = 1 (one column per lane group) / 2 (two columns)
    const char* v = getenv("B200Q_DECAY_ATTN_SPLIT");
    return v ? atoi(v) : 0;
  }();
  const long long pairs = (long long)n_seqs * heads;
  bool two = dim <= 64 && vdim >= 16 && pairs * ((vdim + 15) / 16) >= 2 * 148;
  if (forced == 1 || forced == 2) two = forced == 2 && dim <= 64;
  const int cols = two ? 16 : 8;
  dim3 grid(n_seqs, heads, (vdim + cols - 1) / cols);
  B200Q_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "decay_attn: too many heads or value columns");
#define RECUR_(DT, NC)                                                                                                    \
  do {                                                                                                                   \
    if (w)                                                                                                               \
      decay_attn_kernel<DT, true, NC, 4><<<grid, 32, (size_t)2 * DATT_G * 3 * DT * sizeof(float), st>>>(                 \
          qkv, ldq, q_off, k_off, v_off, head_decay, w, ldw, bonus, state, slot_stride, seq_desc, heads, dim, vdim, raw); \
    else                                                                                                                 \
      decay_attn_kernel<DT, false, NC, 4><<<grid, 32, (size_t)2 * DATT_G * 2 * DT * sizeof(float), st>>>(                \
          qkv, ldq, q_off, k_off, v_off, head_decay, w, ldw, bonus, state, slot_stride, seq_desc, heads, dim, vdim, raw); \
  } while (0)
#define RECUR(DT)            \
  do {                       \
    if (two) RECUR_(DT, 2);  \
    else RECUR_(DT, 1);      \
  } while (0)
  if (dim <= 32) RECUR(32);
  else if (dim <= 64) RECUR(64);
  else if (dim <= 128) RECUR_(128, 1);
  else RECUR_(256, 1);
#undef RECUR_
#undef RECUR
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_gated_rmsnorm(const float* raw, int C, int group, const float* w, const void* gate, int ld_gate, int gate_act,
                        float eps, void* out, int T_, int dtype, void* stream) {
  B200Q_CHECK_ARG(raw && w && gate && out && C > 0 && group > 0 && C % group == 0 && ld_gate >= C &&
                      (gate_act == 0 || gate_act == 1) && eps > 0.f && T_ >= 0 && is_dtype(dtype) && C / group <= 65535,
                  "gated_rmsnorm: bad argument (C=%d group=%d)", C, group);
  if (T_ == 0) return B200Q_OK;
  dim3 grid(T_, C / group);
  const int threads = std::min(256, (group + 31) & ~31);
  DISPATCH_T(dtype, (gated_rmsnorm_kernel<T><<<grid, threads, 0, as_stream(stream)>>>(raw, C, group, w, (const T*)gate,
                                                                                      ld_gate, gate_act, eps, (T*)out)));
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // extern "C"
