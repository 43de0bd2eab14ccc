// dn_seq_recur.cuh -- recurrent mixers with a decay per key channel, and token-shift mixing (libdnet_b200_seq.so).
//
// Both recurrences keep, per head and sequence, an fp32 state M [dk, dv] that every token decays row by row and
// extends by the outer product of its key and value:
//     M_t = diag(d_t) M_(t-1) + k_t v_t^T
// and differ in what the token reads:
//     RECUR_AFTER  (gated linear attention):  o_t = M_t^T q_t
//     RECUR_BONUS  (wkv):                     o_t = (M_(t-1) + diag(u) k_t v_t^T)^T q_t, u a learned bonus per (head, channel)
// q, k, v arrive as projections in the storage type; decays, states and sums are fp32.
#pragma once
#include "dn_seq_kernels.cuh"

namespace dnseq {

constexpr int RECUR_AFTER = 0, RECUR_BONUS = 1;
constexpr int SHIFT_MAX = 5;

// token shift: out_s[n] = h[n] + (h[n-1] - h[n]) mu_s for up to SHIFT_MAX coefficient vectors; the row before an
// entry's first one is the slot's carried row (zeros in a fresh slot).  One block per token.
template <class T>
struct ShiftMu { const T* mu[SHIFT_MAX]; int n; };
template <class T>
__global__ void k_shift_mix(const T* __restrict__ h, Batch b, int W, ShiftMu<T> mu, const T* __restrict__ state, size_t slot_stride,
                            T* __restrict__ out, size_t out_stride) {
  const int n = blockIdx.x;
  const bool has_prev = n > b.first[n];
  const T* prev = has_prev ? h + (size_t)(n - 1) * W : state + (size_t)b.slot[n] * slot_stride;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float x = ldf(h + (size_t)n * W + c), d = ldf(prev + c) - x;
    for (int s = 0; s < mu.n; s++) stf(out + (size_t)s * out_stride + (size_t)n * W + c, x + d * ldf(mu.mu[s] + c));
  }
}
// after the mixes are made: an entry's last row becomes its slot's carried row
template <class T>
__global__ void k_shift_carry(const T* __restrict__ h, Batch b, int W, T* __restrict__ state, size_t slot_stride) {
  const int e = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= W) return;
  state[(size_t)b.ent_slot[e] * slot_stride + c] = h[(size_t)(b.ent_start[e + 1] - 1) * W + c];
}

// between the projections and the recurrence: q (times qscale), k, v to fp32; the decay from its pre-activation
// z [N, C] (in place), C = H dk:
//   RECUR_AFTER: d = sigmoid(z + bias)^(1/tau) = exp(-softplus(-(z + bias)) / tau)
//   RECUR_BONUS: d = exp(-exp(z + bias))
// carry (optional, small steps): the block of an entry's last token also copies the token's mixer input row h[n] to
// the slot's carried row (what k_shift_carry does for large steps; every reader of the old row ran before this kernel)
template <class T>
struct ShiftCarry { const T* h; T* state; size_t slot_stride; int W; const int32_t* first; const int32_t* slot; };
template <class T>
__global__ void k_decay_prep(int mode, int N, int C, int Cv, const T* __restrict__ Uq, const T* __restrict__ Uk, const T* __restrict__ Uv,
                             const T* __restrict__ bias, float qscale, float tau, float* __restrict__ qn, float* __restrict__ kn,
                             float* __restrict__ vv, float* __restrict__ z, ShiftCarry<T> carry) {
  const int n = blockIdx.x;
  if (carry.h && (n == N - 1 || carry.first[n + 1] != carry.first[n])) {
    T* dst = carry.state + (size_t)carry.slot[n] * carry.slot_stride;
    for (int c = threadIdx.x; c < carry.W; c += blockDim.x) dst[c] = carry.h[(size_t)n * carry.W + c];
  }
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const size_t i = (size_t)n * C + c;
    qn[i] = ldf(Uq + i) * qscale;
    kn[i] = ldf(Uk + i);
    const float a = z[i] + ldf(bias + c);
    z[i] = mode == RECUR_AFTER ? expf(-softplus_f(-a) / tau) : expf(-expf(a));
  }
  for (int c = threadIdx.x; c < Cv; c += blockDim.x) vv[(size_t)n * Cv + c] = ldf(Uv + (size_t)n * Cv + c);
}

// The recurrence, token by token.  Columns of M are independent: a block owns COLS columns of one (entry, head); P
// adjacent lanes share a column, each holding R consecutive rows (P R >= dk) in registers.  State
// [slot][head][dk][dv] fp32, read once and written once per step.  A token's k, q, decay and the block's COLS values
// come through shared memory in tiles of TB tokens, copied asynchronously one tile ahead; k, q and the decay lie
// there as P runs of R values, each run padded by 4 floats (the 16-byte reads of a column's P lanes fall into
// different banks); rows from dk up are zero.  The read-out sums a thread's rows in ascending order, then the lanes
// of a column pairwise: an order fixed by (dk, P), whatever the tile size or the cut of a prompt.  U tokens (8 in
// blocks of up to 128 threads, else 4) are taken at a time: their loads are issued ahead, their state updates run back
// to back and their read-outs are reduced together (U independent shuffle chains in flight).
template <int R, int P, int COLS>
__global__ void __launch_bounds__(COLS * P) k_decay_rule(int mode, Batch b, int H, int dk, int dv, int TB, const float* __restrict__ qn,
                                                         const float* __restrict__ kn, const float* __restrict__ vv,
                                                         const float* __restrict__ decay, const void* __restrict__ bonus, int bonus_f32,
                                                         float* __restrict__ state, size_t slot_stride, float* __restrict__ o) {
  static_assert(COLS * P >= 32 && (COLS * P) % 32 == 0 && COLS % 4 == 0 && COLS <= 32, "whole warps, 16-byte rows");
  extern __shared__ __align__(16) float dsm[];      // 2 x TB x per
  constexpr int KP = P * (R + 4);
  constexpr int per = 3 * KP + COLS;                // k q decay v[COLS]
  constexpr int U = COLS * P <= 128 ? 8 : 4;      // tokens a group: as many as the registers of the block size allow
  const int e = blockIdx.x / H, h = blockIdx.x % H;
  const int part = threadIdx.x % P, colb = threadIdx.x / P, col = blockIdx.y * COLS + colb;
  const int s0 = b.ent_start[e], s1 = b.ent_start[e + 1];
  const bool live = col < dv;
  float* Sg = state + (size_t)b.ent_slot[e] * slot_stride + (size_t)h * dk * dv;
  const int r0 = part * R;
  float S[R], u[R];
#pragma unroll
  for (int r = 0; r < R; r++) {
    S[r] = (live && r0 + r < dk) ? Sg[(size_t)(r0 + r) * dv + col] : 0.f;
    u[r] = 0.f;
    if (mode == RECUR_BONUS && r0 + r < dk)
      u[r] = bonus_f32 ? ((const float*)bonus)[(size_t)h * dk + r0 + r] : __bfloat162float(((const bf16*)bonus)[(size_t)h * dk + r0 + r]);
  }
  const int C = H * dk, Cv = H * dv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int nwarp = COLS * P / 32;
  auto stage = [&](int buf, int n0) {
    const int cnt = min(TB, s1 - n0);
    for (int t = warp; t < cnt; t += nwarp) {
      const int n = n0 + t;
      float* dst = dsm + ((size_t)buf * TB + t) * per;
      const size_t base = (size_t)n * C + (size_t)h * dk;
      for (int c = lane; c < P * R; c += 32) {
        const int idx = (c / R) * (R + 4) + (c % R);
        if (c < dk) { cp_async4(dst + idx, kn + base + c); cp_async4(dst + KP + idx, qn + base + c); cp_async4(dst + 2 * KP + idx, decay + base + c); }
        else dst[idx] = dst[KP + idx] = dst[2 * KP + idx] = 0.f;
      }
      if (lane < COLS) {
        const int vc = blockIdx.y * COLS + lane;
        if (vc < dv) cp_async4(dst + 3 * KP + lane, vv + (size_t)n * Cv + h * dv + vc);
        else dst[3 * KP + lane] = 0.f;
      }
    }
    cp_async_commit();
  };
  stage(0, s0);
  int buf = 0;
  for (int n0 = s0; n0 < s1; n0 += TB, buf ^= 1) {
    if (n0 + TB < s1) { stage(buf ^ 1, n0 + TB); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const int cnt = min(TB, s1 - n0);
    for (int t0 = 0; t0 < cnt; t0 += U) {
      float od[U];
      auto token = [&](int uu) {
        const float* in = dsm + ((size_t)buf * TB + t0 + uu) * per;
        const float4* k4 = reinterpret_cast<const float4*>(in + part * (R + 4));
        const float4* q4 = reinterpret_cast<const float4*>(in + KP + part * (R + 4));
        const float4* d4 = reinterpret_cast<const float4*>(in + 2 * KP + part * (R + 4));
        const float v = in[3 * KP + colb];
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < R / 4; j++) {
          const float4 kv = k4[j], qv = q4[j], dv4 = d4[j];
          const float kk[4] = {kv.x, kv.y, kv.z, kv.w}, qq[4] = {qv.x, qv.y, qv.z, qv.w}, dd[4] = {dv4.x, dv4.y, dv4.z, dv4.w};
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const float kvp = kk[i] * v;
            float& Sr = S[4 * j + i];
            if (mode == RECUR_BONUS) {
              acc = fmaf(fmaf(u[4 * j + i], kvp, Sr), qq[i], acc);
              Sr = fmaf(dd[i], Sr, kvp);
            } else {
              Sr = fmaf(dd[i], Sr, kvp);
              acc = fmaf(Sr, qq[i], acc);
            }
          }
        }
        od[uu] = acc;
      };
      if (t0 + U <= cnt) {      // a whole group: no guards, so that the four tokens' loads can be issued ahead of the arithmetic
#pragma unroll
        for (int uu = 0; uu < U; uu++) token(uu);
      } else {
#pragma unroll
        for (int uu = 0; uu < U; uu++) {
          od[uu] = 0.f;
          if (t0 + uu < cnt) token(uu);
        }
      }
#pragma unroll
      for (int x = 1; x < P; x <<= 1) {
#pragma unroll
        for (int uu = 0; uu < U; uu++) od[uu] += __shfl_xor_sync(0xffffffffu, od[uu], x);
      }
      if (live && part == 0) {
#pragma unroll
        for (int uu = 0; uu < U; uu++)
          if (t0 + uu < cnt) o[(size_t)(n0 + t0 + uu) * Cv + h * dv + col] = od[uu];
      }
    }
    __syncthreads();      // the tile is read out before the copy after next lands in it
  }
#pragma unroll
  for (int r = 0; r < R; r++)
    if (live && r0 + r < dk) Sg[(size_t)(r0 + r) * dv + col] = S[r];
}

}  // namespace dnseq
