// Pieces for decoder designs whose mixer runs a softmax attention and a linear attention SIDE BY SIDE on the same
// input, normalises the SUBLAYER'S OUTPUT (not its input) before the residual add, and routes tokens over experts with
// softmax scores, a selection bias, expert groups and identity experts:
//
//   q/k norm + rotary append    per-head weighted RMS norm of q and k, partial rotary with a frequency TABLE (so any
//                               frequency rescaling is the caller's), k and v scattered into the paged pools
//   retention scan              S_t = d_h S_(t-1) + (c k_t) v_t^T,  o_t = S_t^T q_t  with a fixed decay per head, the fp32
//                               state carried per sequence in a slot pool; long portions run as parallel segments
//                               whose missing carry is added afterwards
//   head norm with a gate       o * rsqrt(mean(o^2) + eps) [* w] * act(gate) * out_scale, act = sigmoid or SiLU
//   branch post-norm residual   y = sa a + sb b;  x += ls * w * y * rsqrt(mean(y^2) + eps);  optional copy of x in T
//   grouped softmax routing     softmax scores, choice by score + bias inside the best expert groups, weights = chosen
//                               scores over their sum
//   weighted expert combine     out = sum_k w_k * (expert row | the token's own row for identity experts) + shared row
//
// Every size and constant is a parameter.  Norms, angles, scores, the recurrence and the residual are fp32 (angles are
// formed in double precision from the integer position) whatever the storage dtype T is.  The order of a position's
// sums depends only on the layer's sizes, never on how a batch was cut.
#include <algorithm>
#include <type_traits>

#include "../../include/b200_mixers.h"
#include "b200_common.cuh"

namespace b200 {
namespace {

template <typename F>
int parallel_by_dtype(int dtype, const char* name, F&& f) {
  switch (dtype) {
    case B200_DTYPE_F16:
      return f(static_cast<__half*>(nullptr));
    case B200_DTYPE_BF16:
      return f(static_cast<__nv_bfloat16*>(nullptr));
    case B200_DTYPE_F32:
      return f(static_cast<float*>(nullptr));
    default:
      return fail(B200_EINVAL, "%s: unsupported dtype %d", name, dtype);
  }
}

__device__ __forceinline__ float block_total(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}

__device__ __forceinline__ float sigm(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---- q/k norm + rotary + append ------------------------------------------------------------------------------------
// One CTA per token, one warp per head in turn (q heads, then k heads, then the value rows).  A head's row is read into
// the warp's fp32 slab, normed there, and written out with its rotated pairs.
constexpr int kQkWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kQkWarps * 32)
qknorm_rotary_append_kernel(T* __restrict__ q, int64_t q_stride, const T* __restrict__ k, int64_t k_stride,
                            const T* __restrict__ v, int64_t v_stride, const T* __restrict__ qw, const T* __restrict__ kw,
                            float eps, const double* __restrict__ freqs, int rot_dims, int interleaved,
                            T* __restrict__ k_pool, T* __restrict__ v_pool, const int64_t* __restrict__ slot_mapping,
                            const int32_t* __restrict__ tok_pos, int H, int G, int Gv, int dk, int dv, int block_size) {
  extern __shared__ float qk_sm[];     // cos[rh] sin[rh] slab[warps][dk]
  const int n = blockIdx.x, rh = rot_dims / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* cs = qk_sm;
  float* sn = cs + rh;
  float* slab = sn + rh + warp * dk;
  const double p = static_cast<double>(tok_pos[n]);
  for (int i = threadIdx.x; i < rh; i += blockDim.x) {
    double s, c;
    sincos(p * freqs[i], &s, &c);
    cs[i] = static_cast<float>(c);
    sn[i] = static_cast<float>(s);
  }
  __syncthreads();
  const int64_t slot = slot_mapping[n];
  const int64_t blk = slot >= 0 ? slot / block_size : 0;
  const int off = slot >= 0 ? static_cast<int>(slot - blk * block_size) : 0;
  for (int hh = warp; hh < H + G; hh += kQkWarps) {
    const bool is_q = hh < H;
    if (!is_q && slot < 0) continue;
    const int g = hh - H;
    const T* src = is_q ? q + static_cast<int64_t>(n) * q_stride + hh * dk : k + static_cast<int64_t>(n) * k_stride + g * dk;
    T* dst = is_q ? q + static_cast<int64_t>(n) * q_stride + hh * dk : k_pool + ((blk * G + g) * block_size + off) * dk;
    const T* w = is_q ? qw : kw;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) {
      const float x = Cvt<T>::to_f32(src[i]);
      slab[i] = x;
      ss = fmaf(x, x, ss);
    }
    if (w != nullptr) {
      const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(dk) + eps);
      for (int i = lane; i < dk; i += 32) slab[i] = slab[i] * inv * Cvt<T>::to_f32(w[i]);
    }
    __syncwarp();
    for (int i = lane; i < rh; i += 32) {
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + rh;
      const float u = slab[a], x = slab[b];
      dst[a] = Cvt<T>::from_f32(u * cs[i] - x * sn[i]);
      dst[b] = Cvt<T>::from_f32(x * cs[i] + u * sn[i]);
    }
    for (int i = rot_dims + lane; i < dk; i += 32) dst[i] = Cvt<T>::from_f32(slab[i]);
    __syncwarp();
  }
  if (slot < 0) return;
  const T* vr = v + static_cast<int64_t>(n) * v_stride;
  for (int e = threadIdx.x; e < Gv * dv; e += blockDim.x) {
    const int g = e / dv, i = e - g * dv;
    v_pool[((blk * Gv + g) * block_size + off) * dv + i] = vr[e];
  }
}

// ---- retention scan -------------------------------------------------------------------------------------------------
// One CTA (128 threads) per (sequence, head, 32 value columns).  Four adjacent lanes share a value column; lane r of the
// four keeps the state rows i = r, r + 4, ... of that column in registers for the whole portion.  The inputs of 4 tokens
// are staged in shared memory at a time, double buffered (q and k grouped by r so a thread's rows are contiguous); a
// token costs DK / 4 updates per thread and two shuffles, and a barrier falls once per 4 tokens.
struct RetSeq {
  int tok0, count, slot, fresh;
};
constexpr int kRetChunk = 4;
constexpr int kRetNT = 128;
constexpr int kRetCols = kRetNT / 4;

template <typename T, int DK>
__global__ void __launch_bounds__(kRetNT)
retention_scan_kernel(float* __restrict__ o_raw, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                      int64_t in_stride, const float* __restrict__ decay, float k_scale, float* __restrict__ state,
                      const RetSeq* __restrict__ seqs, int H, int dk, int dv) {
  extern __shared__ __align__(16) float ret_sm[];
  constexpr int RW4 = DK / 4;
  const RetSeq sq = seqs[blockIdx.x];
  const int h = blockIdx.y;
  const int r = threadIdx.x & 3, cl = threadIdx.x >> 2;
  const int col0 = blockIdx.z * kRetCols, col = col0 + cl;
  const bool has_col = col < dv;
  const int ncol = min(kRetCols, dv - col0);
  constexpr int row_len = 2 * DK + kRetCols;
  float* buf0 = ret_sm;
  float* buf1 = ret_sm + kRetChunk * row_len;
  float* st = state + (static_cast<int64_t>(sq.slot) * H + h) * dk * dv;
  const float d = decay[h];
  float S[RW4];
  if (!sq.fresh) {   // the CTA's slab of the state passes shared memory so that global rows move as whole segments
    for (int idx = threadIdx.x; idx < dk * kRetCols; idx += kRetNT) {
      const int i = idx / kRetCols, c = idx - i * kRetCols;
      ret_sm[idx] = c < ncol ? st[i * dv + col0 + c] : 0.f;
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < RW4; ++j) {
    const int i = 4 * j + r;
    S[j] = (!sq.fresh && i < dk) ? ret_sm[i * kRetCols + cl] : 0.f;
  }
  __syncthreads();
  constexpr int kPer = (kRetChunk * row_len + kRetNT - 1) / kRetNT;
  // staged element e = thread + u * 128 of a chunk is (token e / row_len, slot e % row_len); where it comes from does
  // not change from chunk to chunk, so for key sizes whose tables fit in registers the source pointer, the token and
  // the factor (k_scale on key slots) of every element are worked out once
  constexpr bool kTabled = DK <= 128;
  constexpr int kTab = kTabled ? kPer : 1;
  T raw[kPer];
  const T* src[kTab];
  int tok_of[kTab];
  float mul[kTab];
  if constexpr (kTabled) {
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int e = threadIdx.x + u * kRetNT;
      const int tt = e / row_len, sl = e - tt * row_len;
      src[u] = nullptr;
      tok_of[u] = tt;
      mul[u] = (sl >= DK && sl < 2 * DK) ? k_scale : 1.0f;
      if (tt < kRetChunk) {
        const int64_t row = static_cast<int64_t>(sq.tok0 + tt) * in_stride;
        if (sl < 2 * DK) {
          const int s2 = sl < DK ? sl : sl - DK;
          const int i = 4 * (s2 % RW4) + s2 / RW4;
          if (i < dk) src[u] = (sl < DK ? q : k) + row + h * dk + i;
        } else if (sl - 2 * DK < ncol) {
          src[u] = v + row + h * dv + col0 + sl - 2 * DK;
        }
      }
    }
  }
  auto fetch = [&](int t0) {
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      raw[u] = Cvt<T>::from_f32(0.f);
      if constexpr (kTabled) {
        if (src[u] != nullptr && t0 + tok_of[u] < sq.count) raw[u] = src[u][static_cast<int64_t>(t0) * in_stride];
      } else {
        const int e = threadIdx.x + u * kRetNT;
        const int tt = e / row_len, sl = e - tt * row_len;
        if (tt < kRetChunk && t0 + tt < sq.count) {
          const int64_t row = static_cast<int64_t>(sq.tok0 + t0 + tt) * in_stride;
          if (sl < 2 * DK) {
            const int s2 = sl < DK ? sl : sl - DK;
            const int i = 4 * (s2 % RW4) + s2 / RW4;
            if (i < dk) raw[u] = sl < DK ? q[row + h * dk + i] : k[row + h * dk + i];
          } else if (sl - 2 * DK < ncol) {
            raw[u] = v[row + h * dv + col0 + sl - 2 * DK];
          }
        }
      }
    }
  };
  auto commit = [&](float* dst, int n_valid) {
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int e = threadIdx.x + u * kRetNT;
      if constexpr (kTabled) {
        if (tok_of[u] < n_valid) dst[e] = Cvt<T>::to_f32(raw[u]) * mul[u];
      } else {
        const int tt = e / row_len, sl = e - tt * row_len;
        if (tt < n_valid) {
          float val = Cvt<T>::to_f32(raw[u]);
          if (sl >= DK && sl < 2 * DK) val *= k_scale;
          dst[e] = val;
        }
      }
    }
  };
  fetch(0);
  commit(buf0, min(kRetChunk, sq.count));
  __syncthreads();
  for (int t0 = 0; t0 < sq.count; t0 += kRetChunk) {
    const float* cur = ((t0 / kRetChunk) & 1) ? buf1 : buf0;
    float* nxt = ((t0 / kRetChunk) & 1) ? buf0 : buf1;
    const bool more = t0 + kRetChunk < sq.count;
    if (more) fetch(t0 + kRetChunk);
    const int n_here = min(kRetChunk, sq.count - t0);
    for (int tt = 0; tt < n_here; ++tt) {
      const float* row = cur + tt * row_len;
      const float vc = row[2 * DK + cl];
      const float* qr = row + r * RW4;
      const float* kr = row + DK + r * RW4;
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int j = 0; j < RW4; j += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(qr + j);
        const float4 k4 = *reinterpret_cast<const float4*>(kr + j);
        S[j] = fmaf(d, S[j], k4.x * vc);
        o0 = fmaf(S[j], q4.x, o0);
        S[j + 1] = fmaf(d, S[j + 1], k4.y * vc);
        o1 = fmaf(S[j + 1], q4.y, o1);
        S[j + 2] = fmaf(d, S[j + 2], k4.z * vc);
        o0 = fmaf(S[j + 2], q4.z, o0);
        S[j + 3] = fmaf(d, S[j + 3], k4.w * vc);
        o1 = fmaf(S[j + 3], q4.w, o1);
      }
      float o = o0 + o1;
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (r == 0 && has_col) o_raw[(static_cast<int64_t>(sq.tok0 + t0 + tt) * H + h) * dv + col] = o;
    }
    if (more) commit(nxt, min(kRetChunk, sq.count - t0 - kRetChunk));
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < RW4; ++j) {
    const int i = 4 * j + r;
    if (i < dk) ret_sm[i * kRetCols + cl] = S[j];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < dk * kRetCols; idx += kRetNT) {
    const int i = idx / kRetCols, c = idx - i * kRetCols;
    if (c < ncol) st[i * dv + col0 + c] = ret_sm[idx];
  }
}

// ---- retention over long portions: segments in parallel, then the carry ---------------------------------------------
// A long portion is cut into segments that the scan above runs as independent fresh sequences (their end states go to a
// scratch tensor, one slot per segment).  The decay is a constant per head, so what a segment misses is exactly
//   o_t += d^(t - t0 + 1) P^T q_t        with P the true state at the segment's start,
// and P follows from the segments' end states E_j by  P_(j+1) = d^(n_j) P_j + E_j.
// retention_carry: one thread per state element walks a parent's segments, leaves P_j where E_j was and the parent's
// final state in its slot.  parents rows: (first segment, segments, state slot, fresh).
__global__ void __launch_bounds__(256)
retention_carry_kernel(float* __restrict__ state, float* __restrict__ seg_state, const int32_t* __restrict__ parents,
                       const RetSeq* __restrict__ segs, const float* __restrict__ decay, int H, int64_t per_head) {
  const int32_t* pr = parents + 4 * blockIdx.x;
  const int h = blockIdx.y;
  const int64_t e = static_cast<int64_t>(blockIdx.z) * blockDim.x + threadIdx.x;
  if (e >= per_head) return;
  const float d = decay[h];
  float* st = state + (static_cast<int64_t>(pr[2]) * H + h) * per_head + e;
  float P = pr[3] ? 0.f : *st;
  for (int j = 0; j < pr[1]; ++j) {
    float* sp = seg_state + (static_cast<int64_t>(pr[0] + j) * H + h) * per_head + e;
    const float E = *sp;
    *sp = P;
    P = fmaf(powf(d, static_cast<float>(segs[pr[0] + j].count)), P, E);
  }
  *st = P;
}

// retention_apply_carry: one CTA (128 threads) per (segment, head, 32 value columns); the start state's slab sits in
// shared memory, the segment's q rows pass through it 16 tokens at a time; warp w owns tokens 4w .. 4w + 3 of a tile,
// lane c one column.
constexpr int kCarryTok = 16;

template <typename T>
__global__ void __launch_bounds__(128)
retention_apply_carry_kernel(float* __restrict__ o_raw, const T* __restrict__ q, int64_t in_stride,
                             const float* __restrict__ seg_state, const RetSeq* __restrict__ segs,
                             const float* __restrict__ decay, int H, int dk, int dv) {
  extern __shared__ __align__(16) float ca_sm[];
  const RetSeq sg = segs[blockIdx.x];
  const int h = blockIdx.y, col0 = blockIdx.z * 32;
  const int warp = threadIdx.x >> 5, cl = threadIdx.x & 31;
  const int dkp = (dk + 3) & ~3;
  float* P_s = ca_sm;                 // [dkp][32]
  float* q_s = P_s + dkp * 32;        // [kCarryTok][dkp]
  const float* P = seg_state + (static_cast<int64_t>(blockIdx.x) * H + h) * dk * dv;
  for (int idx = threadIdx.x; idx < dkp * 32; idx += blockDim.x) {
    const int i = idx >> 5, c = idx & 31;
    P_s[idx] = (i < dk && col0 + c < dv) ? P[i * dv + col0 + c] : 0.f;
  }
  const float d = decay[h];
  const float d_tile = powf(d, static_cast<float>(kCarryTok));
  float f[4];
#pragma unroll
  for (int jj = 0; jj < 4; ++jj) f[jj] = powf(d, static_cast<float>(warp * 4 + jj + 1));
  for (int t0 = 0; t0 < sg.count; t0 += kCarryTok) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < kCarryTok * dkp; idx += blockDim.x) {
      const int t = idx / dkp, i = idx - t * dkp;
      q_s[idx] = (t0 + t < sg.count && i < dk)
                     ? Cvt<T>::to_f32(q[static_cast<int64_t>(sg.tok0 + t0 + t) * in_stride + h * dk + i]) : 0.f;
    }
    __syncthreads();
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < dkp; i += 4) {
      const float p0 = P_s[i * 32 + cl], p1 = P_s[(i + 1) * 32 + cl], p2 = P_s[(i + 2) * 32 + cl], p3 = P_s[(i + 3) * 32 + cl];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float4 q4 = *reinterpret_cast<const float4*>(q_s + (warp * 4 + jj) * dkp + i);
        acc[jj] = fmaf(p0, q4.x, acc[jj]);
        acc[jj] = fmaf(p1, q4.y, acc[jj]);
        acc[jj] = fmaf(p2, q4.z, acc[jj]);
        acc[jj] = fmaf(p3, q4.w, acc[jj]);
      }
    }
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int t = t0 + warp * 4 + jj;
      if (t < sg.count && col0 + cl < dv) {
        float* o = o_raw + (static_cast<int64_t>(sg.tok0 + t) * H + h) * dv + col0 + cl;
        *o = fmaf(f[jj], acc[jj], *o);
      }
      f[jj] *= d_tile;
    }
  }
}

// ---- head norm with a gate ------------------------------------------------------------------------------------------
// one warp per (token, head) row of fp32 read-outs
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_act_gate_kernel(T* __restrict__ out, int64_t out_stride, const float* __restrict__ x, const T* __restrict__ w,
                          const T* __restrict__ gate, int64_t gate_stride, int gate_act, float out_scale, float eps,
                          int64_t rows, int H, int dv) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float* xr = x + row * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss = fmaf(xr[i], xr[i], ss);
  const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(dv) + eps);
  const int64_t n = row / H;
  const int h = static_cast<int>(row - n * H);
  const T* gr = gate ? gate + n * gate_stride + static_cast<int64_t>(h) * dv : nullptr;
  T* orow = out + n * out_stride + static_cast<int64_t>(h) * dv;
  for (int i = lane; i < dv; i += 32) {
    float y = xr[i] * inv;
    if (w) y *= Cvt<T>::to_f32(w[i]);
    if (gr) {
      const float g = Cvt<T>::to_f32(gr[i]);
      y *= gate_act == 1 ? g * sigm(g) : sigm(g);
    }
    orow[i] = Cvt<T>::from_f32(y * out_scale);
  }
}

// ---- branch post-norm residual --------------------------------------------------------------------------------------
template <typename T, typename A>
__global__ void __launch_bounds__(256)
branch_postnorm_residual_kernel(float* __restrict__ x, const A* __restrict__ a, int64_t a_stride, float sa,
                                const T* __restrict__ b, int64_t b_stride, float sb, const T* __restrict__ w,
                                const T* __restrict__ ls, T* __restrict__ x_out, float eps, int width) {
  extern __shared__ float bp_row[];
  __shared__ float red[32];
  const int64_t n = blockIdx.x;
  const A* ar = a + n * a_stride;
  const T* br = b ? b + n * b_stride : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float y = sa * Cvt<A>::to_f32(ar[i]);
    if (br) y = fmaf(sb, Cvt<T>::to_f32(br[i]), y);
    bp_row[i] = y;
    ss = fmaf(y, y, ss);
  }
  const float inv = rsqrtf(block_total(ss, red) / static_cast<float>(width) + eps);
  float* xr = x + n * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float y = bp_row[i] * inv * Cvt<T>::to_f32(w[i]);
    if (ls) y *= Cvt<T>::to_f32(ls[i]);
    const float s = xr[i] + y;
    xr[i] = s;
    if (x_out) x_out[n * width + i] = Cvt<T>::from_f32(s);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
cast_rows_kernel(T* __restrict__ out, const float* __restrict__ x, int64_t n) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    out[i] = Cvt<T>::from_f32(x[i]);
}

// ---- grouped softmax routing ------------------------------------------------------------------------------------------
// One warp per token.  Shared memory per warp: score[E], choice[E], group best[groups].  Ties go to the lowest index.
constexpr int kRouteWarps = 4;

__device__ __forceinline__ void warp_argmax(float& best, int& bi) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) {
      best = ob;
      bi = oi;
    }
  }
}

__global__ void __launch_bounds__(kRouteWarps * 32)
softmax_group_topk_kernel(int32_t* __restrict__ ids, float* __restrict__ weights, const float* __restrict__ logits,
                          const float* __restrict__ correction, float sum_floor, int n_tok, int E, int top, int groups,
                          int keep) {
  extern __shared__ float rt_sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok = blockIdx.x * kRouteWarps + warp;
  if (tok >= n_tok) return;
  float* score = rt_sm + warp * (2 * E + groups);
  float* choice = score + E;
  float* gbest = choice + E;
  const float* z = logits + static_cast<int64_t>(tok) * E;
  float m = -INFINITY;
  for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
  m = warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float x = expf(z[e] - m);
    score[e] = x;
    sum += x;
  }
  sum = warp_sum(sum);
  for (int e = lane; e < E; e += 32) {
    const float s = score[e] / sum;
    score[e] = s;
    choice[e] = s + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = E / groups;
    for (int g = 0; g < groups; ++g) {
      float b = -INFINITY;
      for (int e = lane; e < per; e += 32) b = fmaxf(b, choice[g * per + e]);
      b = warp_max(b);
      if (lane == 0) gbest[g] = b;
    }
    __syncwarp();
    // the `keep` best groups stay; the others' choice scores become -inf (NaN marks a kept group in gbest)
    for (int r = 0; r < keep; ++r) {
      float b = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float f = gbest[g];
        if (f == f && (f > b || (f == b && g < bi) || bi == 0x7fffffff)) {
          b = f;
          bi = g;
        }
      }
      warp_argmax(b, bi);
      // lanes that saw no candidate carry bi = INT_MAX and b = -inf and lose every comparison above unless all do
      if (lane == 0 && bi != 0x7fffffff) gbest[bi] = __int_as_float(0x7fc00000);
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32) {
      const float f = gbest[e / per];
      if (f == f) choice[e] = -INFINITY;
    }
    __syncwarp();
  }
  float wsum = 0.f;
  for (int r = 0; r < top; ++r) {
    float b = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float f = choice[e];
      if (f == f && (bi == 0x7fffffff || f > b || (f == b && e < bi))) {   // NaN marks an expert already taken
        b = f;
        bi = e;
      }
    }
    // a lane without a candidate must lose: give it the sentinel index and -inf
    warp_argmax(b, bi);
    if (lane == 0) {
      ids[static_cast<int64_t>(tok) * top + r] = bi;
      weights[static_cast<int64_t>(tok) * top + r] = score[bi];
      wsum += score[bi];
      choice[bi] = __int_as_float(0x7fc00000);
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float inv = 1.0f / (wsum + sum_floor);
    for (int r = 0; r < top; ++r) weights[static_cast<int64_t>(tok) * top + r] *= inv;
  }
}

// ---- weighted combine -------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
weighted_expert_combine_kernel(float* __restrict__ out, const T* __restrict__ ys, const int64_t* __restrict__ where,
                               const int32_t* __restrict__ ids, const float* __restrict__ weights,
                               const float* __restrict__ x_self, const T* __restrict__ shared_rows, int top, int n_real,
                               int width) {
  const int64_t n = blockIdx.x;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < top; ++j) {
      const int e = ids[n * top + j];
      const float y = e < n_real ? Cvt<T>::to_f32(ys[where[n * top + j] * width + i]) : x_self[n * width + i];
      a = fmaf(weights[n * top + j], y, a);
    }
    if (shared_rows) a += Cvt<T>::to_f32(shared_rows[n * width + i]);
    out[n * width + i] = a;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_kernel(T* __restrict__ xs, const T* __restrict__ h, const int64_t* __restrict__ src, int top, int width) {
  const T* hr = h + (src[blockIdx.x] / top) * width;
  T* o = xs + static_cast<int64_t>(blockIdx.x) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = hr[i];
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_qknorm_rotary_append(void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v, int64_t v_stride,
                              const void* q_norm, const void* k_norm, float eps, const double* freqs, int rot_dims,
                              int interleaved, void* k_pool, void* v_pool, const int64_t* slot_mapping,
                              const int32_t* tok_pos, int n_tok, int H, int G, int dk, int dv, int block_size,
                              int64_t max_blocks, int dtype, void* stream) {
  return b200_qknorm_rotary_append_ext(q, q_stride, k, k_stride, v, v_stride, q_norm, k_norm, eps, freqs, rot_dims,
                                       interleaved, k_pool, v_pool, slot_mapping, tok_pos, n_tok, H, G, G, dk, dv, block_size,
                                       max_blocks, dtype, stream);
}

int b200_qknorm_rotary_append_ext(void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                                  int64_t v_stride, const void* q_norm, const void* k_norm, float eps, const double* freqs,
                                  int rot_dims, int interleaved, void* k_pool, void* v_pool, const int64_t* slot_mapping,
                                  const int32_t* tok_pos, int n_tok, int H, int G, int Gv, int dk, int dv, int block_size,
                                  int64_t max_blocks, int dtype, void* stream) {
  if (Gv <= 0) return fail(B200_EINVAL, "b200_qknorm_rotary_append: bad sizes");
  if (n_tok < 0 || H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || block_size <= 0 || max_blocks <= 0)
    return fail(B200_EINVAL, "b200_qknorm_rotary_append: bad sizes");
  if (rot_dims < 0 || rot_dims > dk || (rot_dims & 1)) return fail(B200_ESHAPE, "b200_qknorm_rotary_append: rot_dims %d", rot_dims);
  if (n_tok == 0) return 0;
  if (!q || !k || !v || !k_pool || !v_pool || !slot_mapping || !tok_pos || (rot_dims > 0 && !freqs))
    return fail(B200_EINVAL, "b200_qknorm_rotary_append: null pointer");
  const size_t smem = sizeof(float) * (static_cast<size_t>(rot_dims) + static_cast<size_t>(kQkWarps) * dk);
  if (smem > 200 * 1024) return fail(B200_ESHAPE, "b200_qknorm_rotary_append: head size %d too large", dk);
  return parallel_by_dtype(dtype, "b200_qknorm_rotary_append", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto kern = qknorm_rotary_append_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<n_tok, kQkWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(q), q_stride, static_cast<const T*>(k), k_stride, static_cast<const T*>(v), v_stride,
        static_cast<const T*>(q_norm), static_cast<const T*>(k_norm), eps, freqs, rot_dims, interleaved,
        static_cast<T*>(k_pool), static_cast<T*>(v_pool), slot_mapping, tok_pos, H, G, Gv, dk, dv, block_size);
    return check_launch("b200_qknorm_rotary_append");
  });
}

int b200_retention_scan(float* o_raw, const void* q, const void* k, const void* v, int64_t in_stride, const float* decay,
                        float k_scale, float* state, const int32_t* seqs, int n_seqs, int H, int dk, int dv, int dtype,
                        void* stream) {
  if (n_seqs < 0 || H <= 0 || dk <= 0 || dv <= 0) return fail(B200_EINVAL, "b200_retention_scan: bad sizes");
  if (dk > 512) return fail(B200_ESHAPE, "b200_retention_scan: key size %d beyond 512", dk);
  if (n_seqs == 0) return 0;
  if (!o_raw || !q || !k || !v || !decay || !state || !seqs) return fail(B200_EINVAL, "b200_retention_scan: null pointer");
  const int dkt = dk <= 32 ? 32 : (dk <= 64 ? 64 : (dk <= 128 ? 128 : (dk <= 256 ? 256 : 512)));
  const size_t smem = sizeof(float) * std::max<size_t>(2 * kRetChunk * (2 * static_cast<size_t>(dkt) + kRetCols),
                                                       static_cast<size_t>(dk) * kRetCols);
  const dim3 grid(n_seqs, H, (dv + kRetCols - 1) / kRetCols);
  return parallel_by_dtype(dtype, "b200_retention_scan", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto s = static_cast<cudaStream_t>(stream);
    auto launch = [&](auto kern) {
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      kern<<<grid, kRetNT, smem, s>>>(o_raw, static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v),
                                      in_stride, decay, k_scale, state, reinterpret_cast<const RetSeq*>(seqs), H, dk, dv);
    };
    if (dkt == 32) launch(retention_scan_kernel<T, 32>);
    else if (dkt == 64) launch(retention_scan_kernel<T, 64>);
    else if (dkt == 128) launch(retention_scan_kernel<T, 128>);
    else if (dkt == 256) launch(retention_scan_kernel<T, 256>);
    else launch(retention_scan_kernel<T, 512>);
    return check_launch("b200_retention_scan");
  });
}

int b200_retention_carry(float* state, float* seg_state, const int32_t* parents, int n_parents, const int32_t* seg_spans,
                         const float* decay, int H, int dk, int dv, void* stream) {
  if (n_parents < 0 || H <= 0 || dk <= 0 || dv <= 0) return fail(B200_EINVAL, "b200_retention_carry: bad sizes");
  if (n_parents == 0) return 0;
  if (!state || !seg_state || !parents || !seg_spans || !decay) return fail(B200_EINVAL, "b200_retention_carry: null pointer");
  const int64_t per_head = static_cast<int64_t>(dk) * dv;
  const dim3 grid(n_parents, H, static_cast<unsigned>((per_head + 255) / 256));
  retention_carry_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      state, seg_state, parents, reinterpret_cast<const RetSeq*>(seg_spans), decay, H, per_head);
  return check_launch("b200_retention_carry");
}

int b200_retention_apply_carry(float* o_raw, const void* q, int64_t in_stride, const float* seg_state,
                               const int32_t* seg_spans, int n_segs, const float* decay, int H, int dk, int dv, int dtype,
                               void* stream) {
  if (n_segs < 0 || H <= 0 || dk <= 0 || dv <= 0) return fail(B200_EINVAL, "b200_retention_apply_carry: bad sizes");
  if (n_segs == 0) return 0;
  if (!o_raw || !q || !seg_state || !seg_spans || !decay) return fail(B200_EINVAL, "b200_retention_apply_carry: null pointer");
  const int dkp = (dk + 3) & ~3;
  const size_t smem = sizeof(float) * static_cast<size_t>(dkp) * (32 + kCarryTok);
  if (smem > 200 * 1024) return fail(B200_ESHAPE, "b200_retention_apply_carry: key size %d too large", dk);
  const dim3 grid(n_segs, H, (dv + 31) / 32);
  return parallel_by_dtype(dtype, "b200_retention_apply_carry", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto kern = retention_apply_carry_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<grid, 128, smem, static_cast<cudaStream_t>(stream)>>>(o_raw, static_cast<const T*>(q), in_stride, seg_state,
                                                                 reinterpret_cast<const RetSeq*>(seg_spans), decay, H, dk, dv);
    return check_launch("b200_retention_apply_carry");
  });
}

int b200_head_norm_act_gate(void* out, int64_t out_stride, const float* x, const void* weight, const void* gate,
                            int64_t gate_stride, int gate_act, float out_scale, float eps, int64_t n_tok, int H, int dv,
                            int dtype, void* stream) {
  if (n_tok < 0 || H <= 0 || dv <= 0 || gate_act < 0 || gate_act > 1)
    return fail(B200_EINVAL, "b200_head_norm_act_gate: bad sizes");
  if (n_tok == 0) return 0;
  if (!out || !x) return fail(B200_EINVAL, "b200_head_norm_act_gate: null pointer");
  const int64_t rows = n_tok * H;
  return parallel_by_dtype(dtype, "b200_head_norm_act_gate", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    head_norm_act_gate_kernel<T><<<static_cast<unsigned>((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(out), out_stride, x, static_cast<const T*>(weight), static_cast<const T*>(gate), gate_stride,
        gate_act, out_scale, eps, rows, H, dv);
    return check_launch("b200_head_norm_act_gate");
  });
}

int b200_branch_postnorm_residual(float* x, const void* a, int64_t a_stride, int a_is_f32, float sa, const void* b,
                                  int64_t b_stride, float sb, const void* w_norm, const void* layer_scale, void* x_out,
                                  float eps, int rows, int width, int dtype, void* stream) {
  if (rows < 0 || width <= 0 || width > 40000) return fail(B200_EINVAL, "b200_branch_postnorm_residual: bad sizes");
  if (rows == 0) return 0;
  if (!x || !a || !w_norm) return fail(B200_EINVAL, "b200_branch_postnorm_residual: null pointer");
  const size_t smem = static_cast<size_t>(width) * sizeof(float);
  return parallel_by_dtype(dtype, "b200_branch_postnorm_residual", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto s = static_cast<cudaStream_t>(stream);
    auto launch = [&](auto kern, auto* ap) {
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      kern<<<rows, 256, smem, s>>>(x, ap, a_stride, sa, static_cast<const T*>(b), b_stride, sb,
                                   static_cast<const T*>(w_norm), static_cast<const T*>(layer_scale),
                                   static_cast<T*>(x_out), eps, width);
    };
    if (a_is_f32) launch(branch_postnorm_residual_kernel<T, float>, static_cast<const float*>(a));
    else launch(branch_postnorm_residual_kernel<T, T>, static_cast<const T*>(a));
    return check_launch("b200_branch_postnorm_residual");
  });
}

int b200_cast_rows(void* out, const float* x, int64_t n, int dtype, void* stream) {
  if (n < 0) return fail(B200_EINVAL, "b200_cast_rows: bad sizes");
  if (n == 0) return 0;
  if (!out || !x) return fail(B200_EINVAL, "b200_cast_rows: null pointer");
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((n + 255) / 256, kNumSMs * 16));
  return parallel_by_dtype(dtype, "b200_cast_rows", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    cast_rows_kernel<T><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<T*>(out), x, n);
    return check_launch("b200_cast_rows");
  });
}

int b200_softmax_group_topk(int32_t* ids, float* weights, const float* logits, const float* correction, float sum_floor,
                            int n_tok, int E, int top, int groups, int keep, void* stream) {
  if (n_tok < 0 || E <= 0 || top <= 0 || top > E || groups < 1 || keep < 1 || keep > groups || E % groups)
    return fail(B200_EINVAL, "b200_softmax_group_topk: bad sizes");
  if (groups > 1 && keep < groups && static_cast<int64_t>(keep) * (E / groups) < top)
    return fail(B200_EINVAL, "b200_softmax_group_topk: the kept groups hold fewer than `top` experts");
  if (n_tok == 0) return 0;
  if (!ids || !weights || !logits) return fail(B200_EINVAL, "b200_softmax_group_topk: null pointer");
  const size_t smem = sizeof(float) * kRouteWarps * (2 * static_cast<size_t>(E) + groups);
  if (smem > 200 * 1024) return fail(B200_ESHAPE, "b200_softmax_group_topk: %d experts are too many", E);
  auto kern = softmax_group_topk_kernel;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  kern<<<(n_tok + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      ids, weights, logits, correction, sum_floor, n_tok, E, top, groups, keep);
  return check_launch("b200_softmax_group_topk");
}

int b200_gather_rows(void* xs, const void* h, const int64_t* src, int64_t n_rows, int top, int width, int dtype,
                     void* stream) {
  if (n_rows < 0 || top <= 0 || width <= 0) return fail(B200_EINVAL, "b200_gather_rows: bad sizes");
  if (n_rows == 0) return 0;
  if (!xs || !h || !src) return fail(B200_EINVAL, "b200_gather_rows: null pointer");
  return parallel_by_dtype(dtype, "b200_gather_rows", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    gather_rows_kernel<T><<<static_cast<unsigned>(n_rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(xs), static_cast<const T*>(h), src, top, width);
    return check_launch("b200_gather_rows");
  });
}

int b200_weighted_expert_combine(float* out, const void* ys, const int64_t* where, const int32_t* ids, const float* weights,
                                 const float* x_self, const void* shared_rows, int64_t n_tok, int top, int n_real,
                                 int width, int dtype, void* stream) {
  if (n_tok < 0 || top <= 0 || width <= 0 || n_real < 0) return fail(B200_EINVAL, "b200_weighted_expert_combine: bad sizes");
  if (n_tok == 0) return 0;
  if (!out || !where || !ids || !weights || (n_real > 0 && !ys))
    return fail(B200_EINVAL, "b200_weighted_expert_combine: null pointer");
  return parallel_by_dtype(dtype, "b200_weighted_expert_combine", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    weighted_expert_combine_kernel<T><<<static_cast<unsigned>(n_tok), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        out, static_cast<const T*>(ys), where, ids, weights, x_self, static_cast<const T*>(shared_rows), top, n_real, width);
    return check_launch("b200_weighted_expert_combine");
  });
}

}  // extern "C"
