// decay_attn.cu — linear attention with decay: per (sequence, head) an fp32 state S [dim][vdim] that is
// multiplied by a decay and receives the outer product k v^T at every token.  Two forms share one kernel:
//   constant decay per head:          S <- decay_h S + k v^T;   o = S^T q                        (reads the new state)
//   decay per token and key channel:  o = (S + diag(bonus) k v^T)^T q;   S <- diag(w) S + k v^T  (reads the old one)
// followed by a norm over groups of the output row, a weight and a gate (gated_rmsnorm_kernel).
//
// One warp per (sequence, head, 8 value columns): columns of the state are independent, so a head spreads
// over vdim/8 CTAs; four lanes share a column, each with a quarter of it (dim/4 values, zero-padded) in
// registers, partial dot products summed by two butterfly shuffles.  q, k (and w) of 8 tokens at a time arrive
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

constexpr int DATT_G = 8, DATT_COLS = 8;
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

// VECW: decay per token and key channel (with the bonus); else one constant per head
template <int DT, bool VECW>
__global__ void __launch_bounds__(32) decay_attn_kernel(const float* __restrict__ qkv, int ldq, int q_off, int k_off,
                                                        int v_off, const float* __restrict__ head_decay,
                                                        const float* __restrict__ w, int ldw,
                                                        const float* __restrict__ bonus, float* __restrict__ state,
                                                        long long slot_stride, const int32_t* __restrict__ seq_desc,
                                                        int heads, int dim, int vdim, float* __restrict__ raw) {
  constexpr int QL = DT / 4;           // state values per lane
  constexpr int NV = VECW ? 3 : 2;     // vectors per token in shared memory: k, q (, w)
  extern __shared__ __align__(16) float sm[];  // [2][G][NV*DT]
  const SeqView s = seq_view(seq_desc, blockIdx.x);
  if (s.n <= 0) return;
  const int h = blockIdx.y, lane = threadIdx.x, sub = lane >> 3, j = blockIdx.z * DATT_COLS + (lane & 7);
  const int q0 = sub * QL, HV = heads * vdim;
  const bool on = j < vdim;
  const bool vec = (dim & 3) == 0 && (ldq & 3) == 0 && (q_off & 3) == 0 && (k_off & 3) == 0 &&
                   (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 &&
                   (!VECW || ((ldw & 3) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0));
  float* st = state + (long long)s.slot * slot_stride + (long long)h * dim * vdim;
  for (int e = lane; e < 2 * DATT_G * NV * DT; e += 32) sm[e] = 0.f;  // the padding stays zero
  __syncwarp();
  auto fetch = [&](int g0, int buf) {
    const int cnt = min(DATT_G, s.n - g0);
    float* dst0 = sm + (long long)buf * DATT_G * NV * DT;
    if (vec) {
      const int pv = dim / 4, per = NV * pv;  // 16-byte pieces of one token
      for (int e = lane; e < cnt * per; e += 32) {
        const int tk = e / per, pc = e % per, which = pc / pv, off = (pc % pv) * 4;
        const long long row = s.row0 + g0 + tk;
        const float* src = which == 0   ? qkv + row * ldq + k_off + h * dim
                           : which == 1 ? qkv + row * ldq + q_off + h * dim
                                        : w + row * ldw + h * dim;
        cp_async16(dst0 + tk * NV * DT + which * DT + off, src + off);
      }
    } else {
      for (int e = lane; e < cnt * NV * dim; e += 32) {
        const int tk = e / (NV * dim), i = e % (NV * dim), which = i / dim, d = i % dim;
        const long long row = s.row0 + g0 + tk;
        dst0[tk * NV * DT + which * DT + d] = which == 0   ? qkv[row * ldq + k_off + h * dim + d]
                                              : which == 1 ? qkv[row * ldq + q_off + h * dim + d]
                                                           : w[row * ldw + h * dim + d];
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(0, 0);
  float S[QL], U[VECW ? QL : 1];
#pragma unroll
  for (int q = 0; q < QL; ++q) S[q] = (on && q0 + q < dim && s.pos0 > 0) ? st[(long long)(q0 + q) * vdim + j] : 0.f;
  if (VECW) {
#pragma unroll
    for (int q = 0; q < QL; ++q) U[q] = q0 + q < dim ? bonus[h * dim + q0 + q] : 0.f;
  }
  const float lam = VECW ? 1.f : head_decay[h];
  for (int g0 = 0, buf = 0; g0 < s.n; g0 += DATT_G, buf ^= 1) {
    const int cnt = min(DATT_G, s.n - g0);
    float vj[DATT_G];
#pragma unroll
    for (int tk = 0; tk < DATT_G; ++tk)
      vj[tk] = (on && tk < cnt) ? qkv[(long long)(s.row0 + g0 + tk) * ldq + v_off + h * vdim + j] : 0.f;
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
        const float v = vj[tk];
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int q = 0; q < QL / 4; ++q) {
          const float4 k = k4[q], qq = q4[q];
          if (VECW) {
            const float4 ww = w4[q];
            const float a0 = k.x * v, a1 = k.y * v, a2 = k.z * v, a3 = k.w * v;
            o0 = fmaf(fmaf(U[4 * q], a0, S[4 * q]), qq.x, o0);
            o1 = fmaf(fmaf(U[4 * q + 1], a1, S[4 * q + 1]), qq.y, o1);
            o2 = fmaf(fmaf(U[4 * q + 2], a2, S[4 * q + 2]), qq.z, o2);
            o3 = fmaf(fmaf(U[4 * q + 3], a3, S[4 * q + 3]), qq.w, o3);
            S[4 * q] = fmaf(ww.x, S[4 * q], a0);
            S[4 * q + 1] = fmaf(ww.y, S[4 * q + 1], a1);
            S[4 * q + 2] = fmaf(ww.z, S[4 * q + 2], a2);
            S[4 * q + 3] = fmaf(ww.w, S[4 * q + 3], a3);
          } else {
            S[4 * q] = fmaf(lam, S[4 * q], k.x * v);
            S[4 * q + 1] = fmaf(lam, S[4 * q + 1], k.y * v);
            S[4 * q + 2] = fmaf(lam, S[4 * q + 2], k.z * v);
            S[4 * q + 3] = fmaf(lam, S[4 * q + 3], k.w * v);
            o0 = fmaf(S[4 * q], qq.x, o0);
            o1 = fmaf(S[4 * q + 1], qq.y, o1);
            o2 = fmaf(S[4 * q + 2], qq.z, o2);
            o3 = fmaf(S[4 * q + 3], qq.w, o3);
          }
        }
        float o = (o0 + o1) + (o2 + o3);
        o += __shfl_xor_sync(0xffffffffu, o, 8);
        o += __shfl_xor_sync(0xffffffffu, o, 16);
        if (on && sub == 0) raw[(long long)(s.row0 + g0 + tk) * HV + h * vdim + j] = o;
      }
    }
  }
  if (on) {
#pragma unroll
    for (int q = 0; q < QL; ++q)
      if (q0 + q < dim) st[(long long)(q0 + q) * vdim + j] = S[q];
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
  dim3 grid(n_seqs, heads, (vdim + DATT_COLS - 1) / DATT_COLS);
  B200Q_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "decay_attn: too many heads or value columns");
#define RECUR(DT)                                                                                                        \
  do {                                                                                                                   \
    if (w)                                                                                                               \
      decay_attn_kernel<DT, true><<<grid, 32, (size_t)2 * DATT_G * 3 * DT * sizeof(float), st>>>(                        \
          qkv, ldq, q_off, k_off, v_off, head_decay, w, ldw, bonus, state, slot_stride, seq_desc, heads, dim, vdim, raw); \
    else                                                                                                                 \
      decay_attn_kernel<DT, false><<<grid, 32, (size_t)2 * DATT_G * 2 * DT * sizeof(float), st>>>(                       \
          qkv, ldq, q_off, k_off, v_off, head_decay, w, ldw, bonus, state, slot_stride, seq_desc, heads, dim, vdim, raw); \
  } while (0)
  if (dim <= 32) RECUR(32);
  else if (dim <= 64) RECUR(64);
  else if (dim <= 128) RECUR(128);
  else RECUR(256);
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
