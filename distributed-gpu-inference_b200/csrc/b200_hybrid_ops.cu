// Mixers and feed-forward pieces for hybrid decoder designs whose layers read ONE norm of an fp32 residual stream and
// add the mixer's and the feed-forward's outputs to it together:
//
//   RMS norm                    y = x * rsqrt(mean(x^2) + eps) * (offset + w), fp32 or storage-dtype rows in, strided
//   two-branch residual update  x += (a + b), optionally followed by the next layer's input norm
//   xIELU activation            z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2
//   rotary K/V append           partial rotary on q and k, optional rotation of the VALUES over their whole width,
//                               k and v scattered into the paged pools; angles are formed in double precision
//   norm + latent append        RMS-normed latent rows scattered into a one-head pool (keys and values of a latent
//                               attention are the same cached rows)
//   mixed-head paged attention  softmax attention of packed query rows over the paged cache with (all optional) a
//                               sliding window that keeps the first tokens of the sequence, a learned sink logit in
//                               the denominator, a head-mixing matrix applied to the scores before the softmax, a tanh
//                               soft cap on the scores, the inverse value rotation of the output and a per-head
//                               sigmoid gate
//   short causal convolution    per channel over a sequence's tokens, then SiLU; the last taps - 1 inputs of every
//                               live sequence are carried in a slot pool
//   gated delta rule            S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q  with a decay per
//                               key channel, the fp32 state carried per sequence in a slot pool
//   gated head norm             o * rsqrt(mean(o^2) + eps) * w * sigmoid(gate)
//
// Every size and constant of a design is a parameter.  Scores, softmax, norms, decays, the state and the residual
// are fp32 whatever the storage dtype T is.  The order in which a position's sums are formed depends only on that
// position and the layer's sizes, never on how a batch was cut or what else is in it.
#include <algorithm>
#include <type_traits>

#include "../../include/b200_mixers.h"
#include "b200_common.cuh"

namespace b200 {
namespace {

template <typename F>
int hybrid_by_dtype(int dtype, const char* name, F&& f) {
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

__device__ __forceinline__ float block_sum(float v, float* red) {
  // every thread returns the total; `red` holds 32 floats and may be reused after the call's second barrier
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}

__device__ __forceinline__ float sigmoid_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// ---- RMS norm ----------------------------------------------------------------------------------------------------
template <typename T, typename X>
__global__ void __launch_bounds__(256)
rms_norm_kernel(T* __restrict__ out, int64_t out_stride, const X* __restrict__ x, int64_t x_stride,
                const T* __restrict__ w, float w_off, float eps, int width) {
  __shared__ float red[32];
  const X* xr = x + static_cast<int64_t>(blockIdx.x) * x_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = Cvt<X>::to_f32(xr[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = rsqrtf(block_sum(ss, red) / static_cast<float>(width) + eps);
  T* orow = out + static_cast<int64_t>(blockIdx.x) * out_stride;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    orow[i] = Cvt<T>::from_f32(Cvt<X>::to_f32(xr[i]) * inv * (w_off + Cvt<T>::to_f32(w[i])));
}

// ---- x += (a + b); optionally out_next = norm(x; w_next) ---------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
residual_add2_norm_kernel(float* __restrict__ x, const T* __restrict__ a, int64_t a_stride, const T* __restrict__ b,
                          int64_t b_stride, const T* __restrict__ w_next, float w_off, T* __restrict__ out_next,
                          float eps, int width) {
  extern __shared__ float row_s[];
  __shared__ float red[32];
  float* xr = x + static_cast<int64_t>(blockIdx.x) * width;
  const T* ar = a + static_cast<int64_t>(blockIdx.x) * a_stride;
  const T* br = b ? b + static_cast<int64_t>(blockIdx.x) * b_stride : nullptr;
  float sx = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float y = Cvt<T>::to_f32(ar[i]);
    if (br) y += Cvt<T>::to_f32(br[i]);
    const float v = xr[i] + y;
    xr[i] = v;
    row_s[i] = v;
    sx = fmaf(v, v, sx);
  }
  if (w_next == nullptr) return;
  const float inv = rsqrtf(block_sum(sx, red) / static_cast<float>(width) + eps);
  T* orow = out_next + static_cast<int64_t>(blockIdx.x) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    orow[i] = Cvt<T>::from_f32(row_s[i] * inv * (w_off + Cvt<T>::to_f32(w_next[i])));
}

// ---- xIELU -------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
xielu_kernel(T* __restrict__ out, const T* __restrict__ z, int64_t z_stride, const T* __restrict__ pq, int ff, bool vec) {
  // one row per blockIdx.y; 16-byte accesses when the rows allow it
  const float ap = softplus_(Cvt<T>::to_f32(pq[0]));
  const float an = 0.5f + softplus_(Cvt<T>::to_f32(pq[1]));
  const T* zr = z + static_cast<int64_t>(blockIdx.y) * z_stride;
  T* orow = out + static_cast<int64_t>(blockIdx.y) * ff;
  auto act = [&](float v) { return v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v); };
  if (vec) {
    constexpr int E = 16 / sizeof(T);
    for (int c = (blockIdx.x * blockDim.x + threadIdx.x) * E; c < ff; c += gridDim.x * blockDim.x * E) {
      int4 raw = *reinterpret_cast<const int4*>(zr + c);
      T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int u = 0; u < E; ++u) e[u] = Cvt<T>::from_f32(act(Cvt<T>::to_f32(e[u])));
      *reinterpret_cast<int4*>(orow + c) = raw;
    }
  } else {
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < ff; c += gridDim.x * blockDim.x)
      orow[c] = Cvt<T>::from_f32(act(Cvt<T>::to_f32(zr[c])));
  }
}

// ---- rotary K/V append ---------------------------------------------------------------------------------------------
// One CTA per token.  The token's cos / sin tables (rot_dims / 2 entries for q and k, dv / 2 for the values) are
// formed in double precision from the integer position, so a position of any size keeps full fp32 accuracy.
template <typename T>
__global__ void __launch_bounds__(256)
rotary_kv_append_kernel(T* __restrict__ q, int64_t q_stride, const T* __restrict__ k, int64_t k_stride,
                        const T* __restrict__ v, int64_t v_stride, T* __restrict__ k_pool, T* __restrict__ v_pool,
                        const int64_t* __restrict__ slot_mapping, const int32_t* __restrict__ tok_pos, int H, int G, int dk,
                        int dv, int rot_dims, double rot_base, int rotate_values, int interleaved, int block_size,
                        float* __restrict__ value_rot) {
  extern __shared__ float tab[];   // cos_qk[rh] sin_qk[rh] cos_v[vh] sin_v[vh]
  const int n = blockIdx.x;
  const int rh = rot_dims / 2, vh = rotate_values ? dv / 2 : 0;
  float* cq = tab;
  float* sq = cq + rh;
  float* cv = sq + rh;
  float* sv = cv + vh;
  const double p = static_cast<double>(tok_pos[n]);
  for (int i = threadIdx.x; i < rh + vh; i += blockDim.x) {
    const bool is_v = i >= rh;
    const int m = is_v ? i - rh : i;
    const double a = p * pow(rot_base, -2.0 * m / static_cast<double>(is_v ? dv : rot_dims));
    double s, c;
    sincos(a, &s, &c);
    if (is_v) {
      cv[m] = static_cast<float>(c);
      sv[m] = static_cast<float>(s);
      if (value_rot) {   // the attention kernel turns its outputs back with the same numbers
        value_rot[(static_cast<int64_t>(n) * vh + m) * 2] = cv[m];
        value_rot[(static_cast<int64_t>(n) * vh + m) * 2 + 1] = sv[m];
      }
    } else {
      cq[m] = static_cast<float>(c);
      sq[m] = static_cast<float>(s);
    }
  }
  __syncthreads();
  const int64_t slot = slot_mapping[n];
  const int64_t blk = slot >= 0 ? slot / block_size : 0;
  const int off = slot >= 0 ? static_cast<int>(slot - blk * block_size) : 0;
  // q: in place.  a work item is one pair (or one unrotated element, counted past the pairs)
  {
    T* qr = q + static_cast<int64_t>(n) * q_stride;
    const int per = rh + (dk - rot_dims);
    for (int e = threadIdx.x; e < H * per; e += blockDim.x) {
      const int h = e / per, i = e - h * per;
      if (i >= rh) continue;                          // elements past the rotated part stay as they are
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + rh;
      const float u = Cvt<T>::to_f32(qr[h * dk + a]), w = Cvt<T>::to_f32(qr[h * dk + b]);
      qr[h * dk + a] = Cvt<T>::from_f32(u * cq[i] - w * sq[i]);
      qr[h * dk + b] = Cvt<T>::from_f32(w * cq[i] + u * sq[i]);
    }
  }
  if (slot < 0) return;
  {
    const T* kr = k + static_cast<int64_t>(n) * k_stride;
    const int per = rh + (dk - rot_dims);
    for (int e = threadIdx.x; e < G * per; e += blockDim.x) {
      const int g = e / per, i = e - g * per;
      T* dst = k_pool + ((blk * G + g) * block_size + off) * dk;
      if (i >= rh) {
        dst[rot_dims + i - rh] = kr[g * dk + rot_dims + i - rh];
        continue;
      }
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + rh;
      const float u = Cvt<T>::to_f32(kr[g * dk + a]), w = Cvt<T>::to_f32(kr[g * dk + b]);
      dst[a] = Cvt<T>::from_f32(u * cq[i] - w * sq[i]);
      dst[b] = Cvt<T>::from_f32(w * cq[i] + u * sq[i]);
    }
  }
  {
    const T* vr = v + static_cast<int64_t>(n) * v_stride;
    if (rotate_values) {
      for (int e = threadIdx.x; e < G * vh; e += blockDim.x) {
        const int g = e / vh, i = e - g * vh;
        T* dst = v_pool + ((blk * G + g) * block_size + off) * dv;
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + vh;
        const float u = Cvt<T>::to_f32(vr[g * dv + a]), w = Cvt<T>::to_f32(vr[g * dv + b]);
        dst[a] = Cvt<T>::from_f32(u * cv[i] - w * sv[i]);
        dst[b] = Cvt<T>::from_f32(w * cv[i] + u * sv[i]);
      }
      if (dv & 1)   // an odd last element has no partner
        for (int g = threadIdx.x; g < G; g += blockDim.x)
          v_pool[((blk * G + g) * block_size + off) * dv + dv - 1] = vr[g * dv + dv - 1];
    } else {
      for (int e = threadIdx.x; e < G * dv; e += blockDim.x) {
        const int g = e / dv, i = e - g * dv;
        v_pool[((blk * G + g) * block_size + off) * dv + i] = vr[e];
      }
    }
  }
}

// ---- RMS norm + append of a latent row ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
norm_append_kernel(const T* __restrict__ x, int64_t x_stride, const T* __restrict__ w, float w_off, float eps,
                   T* __restrict__ pool, const int64_t* __restrict__ slot_mapping, int width) {
  __shared__ float red[32];
  const T* xr = x + static_cast<int64_t>(blockIdx.x) * x_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = Cvt<T>::to_f32(xr[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = rsqrtf(block_sum(ss, red) / static_cast<float>(width) + eps);
  const int64_t slot = slot_mapping[blockIdx.x];
  if (slot < 0) return;
  T* dst = pool + slot * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    dst[i] = Cvt<T>::from_f32(Cvt<T>::to_f32(xr[i]) * inv * (w_off + Cvt<T>::to_f32(w[i])));
}

// ---- mixed-head paged attention (row form) -------------------------------------------------------------------------
// One CTA per (token, pass of HP heads), four warps.  The keys a position sees are cut into chunks of 32 at absolute
// multiples of 32; the chunks a window skips are never visited.  Warp w takes visible chunks w, w + 4, ... with one key
// per lane for the scores (all heads when a mixing matrix couples them) and one value channel per lane for P.V, keeps a
// running (max, sum, output) per head, and the four partial results are merged through shared memory.  The sink
// logit enters the denominator in the merge.
struct AttnArgs {
  void* out; int64_t out_tok_stride, out_head_stride;
  const void* q; int64_t q_tok_stride, q_head_stride;
  const void* gate; int64_t gate_stride;
  const void* k_pool; const void* v_pool;
  const int32_t* block_tables; int table_stride;
  const int32_t* tok_row; const int32_t* tok_pos;
  const float* talk; const float* sink;
  float scale; int window, keep_first, unrotate, interleaved; double rot_base;
  int H, G, dk, dv, block_size;
  float softcap;   // > 0: score <- softcap * tanh(score / softcap), after the head mixing and before the mask
  int chunk = 0;   // > 0: a position sees only the keys of its own block of `chunk` positions (counted from 0)
  int v_row = 0;   // elements between value rows in v_pool (the value size unless the values are the first columns of wider rows)
  int v_div = 1;   // value head = key head / v_div (several key heads read one value head)
  int row_heads = 0;   // tensor-core kernel, > 0: a tile is ONE token and its 16 rows are consecutive heads of `row_heads`
                       // that share one kv head; H then counts groups of 16 heads
  int out_f32 = 0;     // != 0: `out` is fp32 (same strides, in elements) whatever T is; plain outputs only (no turn back)
  int stage_q = 0;     // tensor-core kernel: a warp's 16 query rows are staged in shared memory once (always with row_heads)
};

// first key a position sees (the kept first tokens of a window aside)
__device__ __forceinline__ int first_visible(const AttnArgs& A, int p) {
  int lo = A.window > 0 ? max(0, p - A.window + 1) : 0;
  if (A.chunk > 0) lo = max(lo, (p / A.chunk) * A.chunk);
  return lo;
}

constexpr int kAttnWarpsRow = 4;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const T* __restrict__ kr, int dk, bool vec) {
  float s = 0.f;
  if (vec) {
    constexpr int E = 16 / sizeof(T);
    for (int d = 0; d < dk; d += E) {
      const int4 raw = *reinterpret_cast<const int4*>(kr + d);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int u = 0; u < E; ++u) s = fmaf(qs[d + u], Cvt<T>::to_f32(e[u]), s);
    }
  } else {
    for (int d = 0; d < dk; ++d) s = fmaf(qs[d], Cvt<T>::to_f32(kr[d]), s);
  }
  return s;
}

template <typename T, int HP, int DVC>
__global__ void __launch_bounds__(kAttnWarpsRow * 32)
mixed_paged_attn_kernel(const AttnArgs A) {
  extern __shared__ __align__(16) float sm[];
  const int n = blockIdx.x, h0 = blockIdx.y * HP;
  const int H = A.H, G = A.G, dk = A.dk, dv = A.dv, bs = A.block_size, rep = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool mixed = A.talk != nullptr;
  const int hs0 = mixed ? 0 : h0;                         // first head whose raw scores are formed here
  const int nhs = mixed ? H : min(HP, H - h0);            // and how many
  float* q_s = sm;                                        // [nhs][dk]
  float* raw_s = q_s + nhs * dk;                          // [warps][nhs][32]
  float* talk_s = raw_s + kAttnWarpsRow * nhs * 32;       // [HP][H]
  float* mrg = talk_s + (mixed ? HP * H : 0);             // [warps][HP][dv + 2], later [HP][dv] of results
  const T* q = static_cast<const T*>(A.q) + static_cast<int64_t>(n) * A.q_tok_stride;
  for (int e = threadIdx.x; e < nhs * dk; e += blockDim.x) {
    const int hh = e / dk, d = e - hh * dk;
    q_s[e] = Cvt<T>::to_f32(q[(hs0 + hh) * A.q_head_stride + d]) * A.scale;
  }
  if (mixed)
    for (int e = threadIdx.x; e < HP * H; e += blockDim.x) {
      const int hl = e / H;
      talk_s[e] = (h0 + hl < H) ? A.talk[(h0 + hl) * H + (e - hl * H)] : 0.f;
    }
  __syncthreads();
  const int p = A.tok_pos[n];
  const int32_t* table = A.block_tables + static_cast<int64_t>(A.tok_row[n]) * A.table_stride;
  const int lo = first_visible(A, p);
  const int kf = A.window > 0 ? min(A.keep_first, lo) : 0;   // kept first tokens that the window no longer covers
  const int Gv = G / A.v_div;
  const int nA = (kf + 31) >> 5;
  const int cB0 = max(nA, lo >> 5), cB1 = p >> 5;
  const int n_chunks = nA + (cB1 - cB0 + 1);
  const T* kp = static_cast<const T*>(A.k_pool);
  const T* vp = static_cast<const T*>(A.v_pool);
  const bool vec = (dk * sizeof(T)) % 16 == 0;
  float m_r[HP], l_r[HP], acc[HP][DVC];
#pragma unroll
  for (int hl = 0; hl < HP; ++hl) {
    m_r[hl] = -INFINITY;
    l_r[hl] = 0.f;
#pragma unroll
    for (int cc = 0; cc < DVC; ++cc) acc[hl][cc] = 0.f;
  }
  float* raw_w = raw_s + warp * nhs * 32;
  for (int idx = warp; idx < n_chunks; idx += kAttnWarpsRow) {
    const int c = idx < nA ? idx : cB0 + idx - nA;
    const int j = c * 32 + lane;
    const bool valid = j <= p && (j >= lo || (A.window > 0 && j < A.keep_first));
    int base = 0, vrow0 = 0;                                 // row of the key / the value in head 0 of its block
    if (valid) {
      const int blk = table[j / bs];
      base = (blk * G) * bs + j % bs;
      vrow0 = (blk * Gv) * bs + j % bs;
    }
    __syncwarp();
    if (valid) {
      for (int hh = 0; hh < nhs; ++hh) {
        const int g = (hs0 + hh) / rep;
        raw_w[hh * 32 + lane] = dot_row<T>(q_s + hh * dk, kp + static_cast<int64_t>(base + g * bs) * dk, dk, vec);
      }
    }
    __syncwarp();
    float pr[HP];
#pragma unroll
    for (int hl = 0; hl < HP; ++hl) {
      pr[hl] = 0.f;
      if (h0 + hl < H) {          // uniform over the warp
        float t = -INFINITY;
        if (valid) {
          if (mixed) {
            t = 0.f;
            for (int g = 0; g < H; ++g) t = fmaf(talk_s[hl * H + g], raw_w[g * 32 + lane], t);
          } else {
            t = raw_w[hl * 32 + lane];
          }
          if (A.softcap > 0.f) t = A.softcap * tanhf(t / A.softcap);
        }
        const float m_new = fmaxf(m_r[hl], warp_max(t));
        if (m_new != -INFINITY) {
          const float corr = expf(m_r[hl] - m_new);          // exp(-inf) = 0 for the first chunk with a visible key
          const float e = valid ? expf(t - m_new) : 0.f;
          l_r[hl] = l_r[hl] * corr + warp_sum(e);
          m_r[hl] = m_new;
          pr[hl] = e;
#pragma unroll
          for (int cc = 0; cc < DVC; ++cc) acc[hl][cc] *= corr;
        }
      }
    }
    for (int jj = 0; jj < 32; ++jj) {
      const int vbase = __shfl_sync(0xffffffffu, vrow0, jj);
      float vv[DVC];
      int g_have = -1;
#pragma unroll
      for (int hl = 0; hl < HP; ++hl) {
        const float pj = __shfl_sync(0xffffffffu, pr[hl], jj);
        if (pj != 0.f) {         // uniform over the warp; also skips heads past H and keys that are masked
          const int g = (h0 + hl) / rep / A.v_div;
          if (g != g_have) {
            const T* vr = vp + static_cast<int64_t>(vbase + g * bs) * A.v_row;
#pragma unroll
            for (int cc = 0; cc < DVC; ++cc) vv[cc] = (lane + 32 * cc < dv) ? Cvt<T>::to_f32(vr[lane + 32 * cc]) : 0.f;
            g_have = g;
          }
#pragma unroll
          for (int cc = 0; cc < DVC; ++cc) acc[hl][cc] = fmaf(pj, vv[cc], acc[hl][cc]);
        }
      }
    }
  }
  // merge the warps' partial results
  const int mw = dv + 2;
#pragma unroll
  for (int hl = 0; hl < HP; ++hl) {
    float* dst = mrg + (warp * HP + hl) * mw;
#pragma unroll
    for (int cc = 0; cc < DVC; ++cc)
      if (lane + 32 * cc < dv) dst[lane + 32 * cc] = acc[hl][cc];
    if (lane == 0) { dst[dv] = m_r[hl]; dst[dv + 1] = l_r[hl]; }
  }
  __syncthreads();
  float* res = raw_s;    // [HP][dv] — the score staging area is free now (nhs * 128 >= HP * dv is checked on the host)
  for (int e = threadIdx.x; e < HP * dv; e += blockDim.x) {
    const int hl = e / dv, c = e - hl * dv;
    if (h0 + hl >= H) continue;
    float M = A.sink ? A.sink[h0 + hl] : -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarpsRow; ++w) M = fmaxf(M, mrg[(w * HP + hl) * mw + dv]);
    float L = A.sink ? expf(A.sink[h0 + hl] - M) : 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarpsRow; ++w) {
      const float* src = mrg + (w * HP + hl) * mw;
      const float f = src[dv] == -INFINITY ? 0.f : expf(src[dv] - M);
      L = fmaf(src[dv + 1], f, L);
      O = fmaf(src[c], f, O);
    }
    res[e] = O / L;
  }
  __syncthreads();
  T* out = static_cast<T*>(A.out) + static_cast<int64_t>(n) * A.out_tok_stride;
  const T* gate = static_cast<const T*>(A.gate);
  if (A.unrotate) {
    const int vh = dv / 2;
    for (int e = threadIdx.x; e < HP * vh; e += blockDim.x) {
      const int hl = e / vh, i = e - hl * vh;
      if (h0 + hl >= H) continue;
      double s, c;
      sincos(static_cast<double>(p) * pow(A.rot_base, -2.0 * i / static_cast<double>(dv)), &s, &c);
      const float cf = static_cast<float>(c), sf = static_cast<float>(s);
      const int a = A.interleaved ? 2 * i : i, b = A.interleaved ? 2 * i + 1 : i + vh;
      const float u = res[hl * dv + a], w = res[hl * dv + b];
      float ya = u * cf + w * sf, yb = w * cf - u * sf;        // the rotation by -p
      if (gate) {
        const float gt = sigmoid_(Cvt<T>::to_f32(gate[static_cast<int64_t>(n) * A.gate_stride + h0 + hl]));
        ya *= gt; yb *= gt;
      }
      T* orow = out + (h0 + hl) * A.out_head_stride;
      orow[a] = Cvt<T>::from_f32(ya);
      orow[b] = Cvt<T>::from_f32(yb);
    }
    if (dv & 1)
      for (int hl = threadIdx.x; hl < HP; hl += blockDim.x)
        if (h0 + hl < H) out[(h0 + hl) * A.out_head_stride + dv - 1] = Cvt<T>::from_f32(res[hl * dv + dv - 1]);
  } else {
    for (int e = threadIdx.x; e < HP * dv; e += blockDim.x) {
      const int hl = e / dv, c = e - hl * dv;
      if (h0 + hl >= H) continue;
      float y = res[e];
      if (gate) y *= sigmoid_(Cvt<T>::to_f32(gate[static_cast<int64_t>(n) * A.gate_stride + h0 + hl]));
      if (A.out_f32) static_cast<float*>(A.out)[static_cast<int64_t>(n) * A.out_tok_stride + (h0 + hl) * A.out_head_stride + c] = y;
      else out[(h0 + hl) * A.out_head_stride + c] = Cvt<T>::from_f32(y);
    }
  }
}

// ---- mixed-head paged attention on the tensor cores (16-bit storage types) -----------------------------------------
// A CTA serves up to 16 consecutive tokens of one sequence (one m16 row block) and up to 8 * HW query heads: warp w
// owns heads w * HW .. w * HW + HW - 1 of the CTA's range.  Keys are walked in tiles of 32 at absolute multiples of 32,
// skipping the tiles a window hides; the K and V rows of a tile (every kv head the CTA needs) arrive in shared memory
// by cp.async with zero fill past the sequence's end.  S = Q K^T and O += P V are mma.sync m16n8k16 with fp32
// accumulators; the softmax runs in fp32 on the S fragments and only the weights P are rounded to the storage type as
// the left operand of P V.  With a head-mixing matrix the CTA's warps first form the raw scores of ALL heads into
// shared memory and every warp then mixes the rows of its own heads from there.  When keys and values are the same
// pool (a latent attention) and equally wide, one staged tile serves both products.  Outputs that have to be turned
// back pass a per-warp fp32 slab in shared memory, where a pair's two halves meet.
template <typename T>
struct Mma16x8;
template <>
struct Mma16x8<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
};
template <>
struct Mma16x8<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
};

__device__ __forceinline__ void stage16(void* smem_dst, const void* gmem_src, bool valid) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  const int bytes = valid ? 16 : 0;   // no source bytes: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}

// c * tanh(s / c) as c * (1 - 2 / (exp(2 s / c) + 1)) with the hardware exponential and reciprocal: absolute error of a
// few 1e-7 * c, far below the rounding of the 16-bit weights the scores turn into (two_over_c = 2 / c)
__device__ __forceinline__ float soft_cap(float s, float c, float two_over_c) {
  return c * (1.0f - __fdividef(2.0f, __expf(s * two_over_c) + 1.0f));
}

constexpr int kTcWarps = 8;
constexpr int kTcKeys = 32;
constexpr int kTcRows = 16;
constexpr int kTcRawStride = 40;

// EXT: the kernel also knows blocks of positions, values inside wider rows or shared by several key heads, and heads on
// the rows; layers without any of these run the instantiation that carries none of it.
template <typename T, int DV8, int HW, bool EXT>
__global__ void __launch_bounds__(kTcWarps * 32, (HW == 1 && DV8 <= 16) ? 2 : 1)
mixed_prompt_attn_kernel(const AttnArgs A, const int32_t* __restrict__ tiles, const float* __restrict__ rot_tab,
                         float* __restrict__ ws, int n_tok, int stages) {
  extern __shared__ __align__(16) unsigned char tc_smem[];
  constexpr int HC = kTcWarps * HW;
  constexpr int DVP = DV8 * 8;
  const int row0 = tiles[3 * blockIdx.x], cnt = tiles[3 * blockIdx.x + 1], trow = tiles[3 * blockIdx.x + 2];
  const int H = A.H, G = A.G, dk = A.dk, dv = A.dv, bs = A.block_size, rep = H / G;
  const int h0 = blockIdx.y * HC;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, qr = lane >> 2, qc = (lane & 3) * 2;
  const bool mixed = A.talk != nullptr;
  const int g_lo = mixed ? 0 : h0 / rep;
  const int Gs = (mixed ? G - 1 : min(H - 1, h0 + HC - 1) / rep) - g_lo + 1;   // kv heads staged per tile
  const T* kp = static_cast<const T*>(A.k_pool);
  const T* vp = static_cast<const T*>(A.v_pool);
  const int v_div = EXT ? A.v_div : 1, v_row = EXT ? A.v_row : dv;
  const bool alias = (A.v_pool == A.k_pool) && v_div == 1 && DVP <= dk;   // the values are the first columns of the staged key rows
  const int ks = dk + 8, vs = alias ? ks : DVP + 8;                             // row strides in elements
  const int Gv = G / v_div;
  auto first_seen = [&](int p) {     // first key a position sees (the kept first tokens of a window aside)
    int lo = A.window > 0 ? max(0, p - A.window + 1) : 0;
    if (EXT && A.chunk > 0) lo = max(lo, (p / A.chunk) * A.chunk);
    return lo;
  };
  const int stage_elems = Gs * kTcKeys * (ks + (alias ? 0 : vs));                 // one stage: K rows, then V rows
  T* stage0 = reinterpret_cast<T*>(tc_smem);
  const T* Ks = stage0;                                                         // the stage being computed on
  const T* Vs = alias ? stage0 : stage0 + Gs * kTcKeys * ks;
  float* raw = reinterpret_cast<float*>(stage0 + stages * stage_elems);         // [H][16][40]
  float* talk_s = raw + (mixed ? H * kTcRows * kTcRawStride : 0);                               // [HC][H]
  const int RH = EXT ? A.row_heads : 0;
  // a warp's 16 query rows staged once: few resident warps cannot hide the latency of re-reading them for every key tile
  // (heads on the rows: one warp per CTA; wide value layouts: one CTA per SM)
  const bool QS = EXT && A.stage_q;
  T* q_s = reinterpret_cast<T*>(talk_s + (mixed ? HC * H : 0));                                 // [HC][16][dk + 8]
  if (QS) {
    const int kch = dk / 8;
    for (int hl = warp * HW; hl < warp * HW + HW; ++hl) {
      const int h = h0 + hl;
      if (h >= H) continue;
      for (int e = lane; e < kTcRows * kch; e += 32) {
        const int r = e / kch, ch = e - r * kch;
        int4 v = make_int4(0, 0, 0, 0);
        const bool ok = RH ? 16 * h + r < RH : r < cnt;
        if (ok)
          v = *reinterpret_cast<const int4*>(static_cast<const T*>(A.q) +
                                             (RH ? static_cast<int64_t>(row0) * A.q_tok_stride + (16 * h + r) * A.q_head_stride
                                                 : static_cast<int64_t>(row0 + r) * A.q_tok_stride + h * A.q_head_stride) + ch * 8);
        *reinterpret_cast<int4*>(q_s + (hl * kTcRows + r) * ks + ch * 8) = v;
      }
    }
  }
  const int p0 = A.tok_pos[row0], p_last = RH ? p0 : p0 + cnt - 1;
  const int32_t* table = A.block_tables + static_cast<int64_t>(trow) * A.table_stride;
  const int lo0 = first_seen(p0);
  const int kf = A.window > 0 ? min(A.keep_first, lo0) : 0;
  const int nA = (kf + kTcKeys - 1) / kTcKeys;
  const int cB0 = max(nA, lo0 / kTcKeys), cB1 = p_last / kTcKeys;
  const int n_tiles = nA + (cB1 - cB0 + 1);
  if (mixed)
    for (int e = threadIdx.x; e < HC * H; e += blockDim.x) {
      const int hl = e / H;
      talk_s[e] = (h0 + hl < H) ? A.talk[(h0 + hl) * H + (e - hl * H)] : 0.f;
    }
  if (!alias && dv < DVP)     // value columns past dv are never staged: they stay zero
    for (int e = threadIdx.x; e < stages * Gs * kTcKeys * (DVP - dv); e += blockDim.x) {
      const int sgi = e / (Gs * kTcKeys * (DVP - dv)), e2 = e - sgi * (Gs * kTcKeys * (DVP - dv));
      const int r = e2 / (DVP - dv), c = e2 - r * (DVP - dv);
      stage0[sgi * stage_elems + Gs * kTcKeys * ks + r * vs + dv + c] = Cvt<T>::from_f32(0.f);
    }
  float m_r[HW][2], l_r[HW][2], O[HW][DV8][4];
#pragma unroll
  for (int hw = 0; hw < HW; ++hw) {
    m_r[hw][0] = m_r[hw][1] = -INFINITY;
    l_r[hw][0] = l_r[hw][1] = 0.f;
#pragma unroll
    for (int nt = 0; nt < DV8; ++nt) O[hw][nt][0] = O[hw][nt][1] = O[hw][nt][2] = O[hw][nt][3] = 0.f;
  }
  const T* qbase = static_cast<const T*>(A.q);
  const float cap2 = A.softcap > 0.f ? 2.0f / A.softcap : 0.f;
  // S fragments of one head against the staged K tile; rows past the tile's tokens read zeros
  auto scores = [&](int h, float (&s)[4][4]) {
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    // the staged rows (rows past the tile's are zero), else the query rows in global memory
    const T* qa = QS ? q_s + ((h - h0) * kTcRows + qr) * ks + qc
                     : qbase + static_cast<int64_t>(row0 + qr) * A.q_tok_stride + h * A.q_head_stride + qc;
    const T* qb = qa + 8 * (QS ? static_cast<int64_t>(ks) : A.q_tok_stride);
    const int rows = RH ? min(16, RH - 16 * h) : cnt;
    const bool va = qr < rows, vb = qr + 8 < rows;
    const T* kt = Ks + (h / rep - g_lo) * kTcKeys * ks + qr * ks + qc;
    for (int kk = 0; kk < dk; kk += 16) {
      uint32_t a[4];
      a[0] = va ? *reinterpret_cast<const uint32_t*>(qa + kk) : 0u;
      a[1] = vb ? *reinterpret_cast<const uint32_t*>(qb + kk) : 0u;
      a[2] = va ? *reinterpret_cast<const uint32_t*>(qa + kk + 8) : 0u;
      a[3] = vb ? *reinterpret_cast<const uint32_t*>(qb + kk + 8) : 0u;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kt + nt * 8 * ks + kk);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kt + nt * 8 * ks + kk + 8);
        Mma16x8<T>::mma(s[nt], a, b0, b1);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] *= A.scale;
  };
  // the K and V rows of key tile `it` into stage `b` (cp.async; rows past the sequence's end are zero-filled)
  auto issue = [&](int it, int b) {
    const int j0 = (it < nA ? it : cB0 + it - nA) * kTcKeys;
    T* Kd = stage0 + b * stage_elems;
    T* Vd = Kd + Gs * kTcKeys * ks;
    const int kch = dk / 8;
    for (int e = threadIdx.x; e < Gs * kTcKeys * kch; e += blockDim.x) {
      const int ch = e % kch, r = e / kch, key = r % kTcKeys, gi = r / kTcKeys, j = j0 + key;
      const bool ok = j <= p_last;
      const T* src = ok ? kp + (static_cast<int64_t>(table[j / bs] * G + g_lo + gi) * bs + j % bs) * dk + ch * 8 : kp;
      stage16(Kd + r * ks + ch * 8, src, ok);
    }
    if (!alias) {
      const int vch = dv / 8;
      for (int e = threadIdx.x; e < Gs * kTcKeys * vch; e += blockDim.x) {
        const int ch = e % vch, r = e / vch, key = r % kTcKeys, gi = r / kTcKeys, j = j0 + key;
        const bool ok = j <= p_last;
        const T* src = ok ? vp + (static_cast<int64_t>(table[j / bs] * Gv + (g_lo + gi) / v_div) * bs + j % bs) * v_row + ch * 8 : vp;
        stage16(Vd + r * vs + ch * 8, src, ok);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // this CTA's share of the key tiles (gridDim.z > 1: steps of few tokens split the keys over CTAs)
  const int per_split = (n_tiles + gridDim.z - 1) / gridDim.z;
  const int it_lo = blockIdx.z * per_split, it_hi = min(n_tiles, it_lo + per_split);
  __syncthreads();
  if (it_lo < it_hi) issue(it_lo, 0);
  for (int it = it_lo; it < it_hi; ++it) {
    const int j0 = (it < nA ? it : cB0 + it - nA) * kTcKeys;
    const int b = stages == 2 ? ((it - it_lo) & 1) : 0;
    if (stages == 2 && it + 1 < it_hi) {
      issue(it + 1, b ^ 1);       // that stage was last read one iteration ago, before the barrier that ended it
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    Ks = stage0 + b * stage_elems;
    Vs = alias ? Ks : Ks + Gs * kTcKeys * ks;
    if (mixed) {
      for (int g = warp; g < H; g += kTcWarps) {
        float s[4][4];
        scores(g, s);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          float* dst = raw + (g * kTcRows + qr) * kTcRawStride + nt * 8 + qc;
          *reinterpret_cast<float2*>(dst) = make_float2(s[nt][0], s[nt][1]);
          *reinterpret_cast<float2*>(dst + 8 * kTcRawStride) = make_float2(s[nt][2], s[nt][3]);
        }
      }
      __syncthreads();
    }
#pragma unroll
    for (int hw = 0; hw < HW; ++hw) {
      const int hl = warp * HW + hw, h = h0 + hl;
      if (h >= H) continue;      // uniform over the warp
      float s[4][4];
      if (mixed) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        for (int g = 0; g < H; ++g) {
          const float tw = talk_s[hl * H + g];
          const float* src = raw + (g * kTcRows + qr) * kTcRawStride + qc;
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) {
            const float2 lo = *reinterpret_cast<const float2*>(src + nt * 8);
            const float2 hi = *reinterpret_cast<const float2*>(src + 8 * kTcRawStride + nt * 8);
            s[nt][0] = fmaf(tw, lo.x, s[nt][0]);
            s[nt][1] = fmaf(tw, lo.y, s[nt][1]);
            s[nt][2] = fmaf(tw, hi.x, s[nt][2]);
            s[nt][3] = fmaf(tw, hi.y, s[nt][3]);
          }
        }
      } else {
        scores(h, s);
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = qr + 8 * half, p = RH ? p0 : p0 + row;
        const bool row_ok = row < (RH ? min(16, RH - 16 * h) : cnt);
        const int lo_p = first_seen(p);
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = j0 + nt * 8 + qc + e;
            const bool ok = row_ok && j <= p && (j >= lo_p || (A.window > 0 && j < A.keep_first));
            if (A.softcap > 0.f) s[nt][2 * half + e] = soft_cap(s[nt][2 * half + e], A.softcap, cap2);
            if (!ok) s[nt][2 * half + e] = -INFINITY;
            mx = fmaxf(mx, s[nt][2 * half + e]);
          }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_r[hw][half], mx);
        float corr = 1.f, sum = 0.f;
        if (m_new == -INFINITY) {        // nothing visible for this row yet: all weights are zero
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) s[nt][2 * half] = s[nt][2 * half + 1] = 0.f;
        } else {
          corr = expf(m_r[hw][half] - m_new);
#pragma unroll
          for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float w = expf(s[nt][2 * half + e] - m_new);   // exp(-inf) = 0 for hidden keys
              s[nt][2 * half + e] = w;
              sum += w;
            }
          m_r[hw][half] = m_new;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l_r[hw][half] = l_r[hw][half] * corr + sum;
#pragma unroll
        for (int nt = 0; nt < DV8; ++nt) {
          O[hw][nt][2 * half] *= corr;
          O[hw][nt][2 * half + 1] *= corr;
        }
      }
      const T* vt = Vs + ((h / rep - g_lo) * kTcKeys + (lane & 15)) * vs;
#pragma unroll
      for (int kst = 0; kst < 2; ++kst) {
        uint32_t a[4];
        a[0] = Mma16x8<T>::pack(s[2 * kst][0], s[2 * kst][1]);
        a[1] = Mma16x8<T>::pack(s[2 * kst][2], s[2 * kst][3]);
        a[2] = Mma16x8<T>::pack(s[2 * kst + 1][0], s[2 * kst + 1][1]);
        a[3] = Mma16x8<T>::pack(s[2 * kst + 1][2], s[2 * kst + 1][3]);
#pragma unroll
        for (int nt = 0; nt < DV8; ++nt) {
          uint32_t b0, b1;
          const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(vt + kst * 16 * vs + nt * 8));
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
          Mma16x8<T>::mma(O[hw][nt], a, b0, b1);
        }
      }
    }
    __syncthreads();          // the tile (and the raw scores) have been consumed
    if (stages == 1 && it + 1 < it_hi) issue(it + 1, 0);
  }
  if (gridDim.z > 1) {
    // partial (max, sum, unnormalised output) of this CTA's keys; the combine kernel merges the splits
#pragma unroll
    for (int hw = 0; hw < HW; ++hw) {
      const int h = h0 + warp * HW + hw;
      if (h >= H) continue;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = qr + 8 * half;
        if (row >= (RH ? min(16, RH - 16 * h) : cnt)) continue;
        float* dst = RH ? ws + ((static_cast<int64_t>(blockIdx.z) * n_tok + row0) * RH + 16 * h + row) * (DVP + 2)
                        : ws + ((static_cast<int64_t>(blockIdx.z) * n_tok + row0 + row) * H + h) * (DVP + 2);
        if (qc == 0) {
          dst[0] = m_r[hw][half];
          dst[1] = l_r[hw][half];
        }
#pragma unroll
        for (int nt = 0; nt < DV8; ++nt)
          *reinterpret_cast<float2*>(dst + 2 + nt * 8 + qc) = make_float2(O[hw][nt][2 * half], O[hw][nt][2 * half + 1]);
      }
    }
    return;
  }
  __syncthreads();     // the staging area becomes the warps' output slabs
  float* slab = reinterpret_cast<float*>(tc_smem) + warp * kTcRows * DVP;
  T* outp = static_cast<T*>(A.out);
  const T* gate = static_cast<const T*>(A.gate);
#pragma unroll
  for (int hw = 0; hw < HW; ++hw) {
    const int h = h0 + warp * HW + hw;
    if (h >= H) continue;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = qr + 8 * half;
      float f = 0.f;
      if (row < (RH ? min(16, RH - 16 * h) : cnt)) {
        float m = m_r[hw][half], l = l_r[hw][half];
        if (A.sink) {
          const float sk = A.sink[RH ? 16 * h + row : h], M = fmaxf(m, sk);
          l = l * expf(m - M) + expf(sk - M);
          f = expf(m - M) / l;
        } else {
          f = 1.0f / l;
        }
        if (gate && !A.unrotate) f *= sigmoid_(Cvt<T>::to_f32(gate[static_cast<int64_t>(row0 + row) * A.gate_stride + h]));
      }
#pragma unroll
      for (int nt = 0; nt < DV8; ++nt) {
        O[hw][nt][2 * half] *= f;
        O[hw][nt][2 * half + 1] *= f;
      }
    }
    if (!A.unrotate) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = qr + 8 * half;
        if (row >= (RH ? min(16, RH - 16 * h) : cnt)) continue;
        T* orow = RH ? outp + static_cast<int64_t>(row0) * A.out_tok_stride + (16 * h + row) * A.out_head_stride
                     : outp + static_cast<int64_t>(row0 + row) * A.out_tok_stride + h * A.out_head_stride;
#pragma unroll
        for (int nt = 0; nt < DV8; ++nt) {
          const int c = nt * 8 + qc;
          if (c >= dv) continue;
          if (EXT && A.out_f32)
            *reinterpret_cast<float2*>(static_cast<float*>(A.out) + (orow - outp) + c) = make_float2(O[hw][nt][2 * half], O[hw][nt][2 * half + 1]);
          else
            *reinterpret_cast<uint32_t*>(orow + c) = Mma16x8<T>::pack(O[hw][nt][2 * half], O[hw][nt][2 * half + 1]);
        }
      }
    } else {
      __syncwarp();
#pragma unroll
      for (int nt = 0; nt < DV8; ++nt) {
        slab[qr * DVP + nt * 8 + qc] = O[hw][nt][0];
        slab[qr * DVP + nt * 8 + qc + 1] = O[hw][nt][1];
        slab[(qr + 8) * DVP + nt * 8 + qc] = O[hw][nt][2];
        slab[(qr + 8) * DVP + nt * 8 + qc + 1] = O[hw][nt][3];
      }
      __syncwarp();
      const int vh = dv / 2;
      for (int e = lane; e < cnt * vh; e += 32) {
        const int row = e / vh, i = e - row * vh;
        const float cf = rot_tab[(static_cast<int64_t>(row0 + row) * vh + i) * 2];
        const float sf = rot_tab[(static_cast<int64_t>(row0 + row) * vh + i) * 2 + 1];
        const int a = A.interleaved ? 2 * i : i, b = A.interleaved ? 2 * i + 1 : i + vh;
        const float u = slab[row * DVP + a], w = slab[row * DVP + b];
        float ya = u * cf + w * sf, yb = w * cf - u * sf;       // the rotation by minus the position
        if (gate) {
          const float gt = sigmoid_(Cvt<T>::to_f32(gate[static_cast<int64_t>(row0 + row) * A.gate_stride + h]));
          ya *= gt;
          yb *= gt;
        }
        T* orow = outp + static_cast<int64_t>(row0 + row) * A.out_tok_stride + h * A.out_head_stride;
        orow[a] = Cvt<T>::from_f32(ya);
        orow[b] = Cvt<T>::from_f32(yb);
      }
      if (dv & 1)
        for (int row = lane; row < cnt; row += 32)
          outp[static_cast<int64_t>(row0 + row) * A.out_tok_stride + h * A.out_head_stride + dv - 1] =
              Cvt<T>::from_f32(slab[row * DVP + dv - 1]);
    }
  }
}

// Merge of the key splits: one CTA per token.  out(h) = sum_s O_s e^(m_s - M) / (sum_s l_s e^(m_s - M) + e^(sink - M)),
// then the turn back and the gate, as in the single-CTA epilogue.
template <typename T>
__global__ void __launch_bounds__(256)
attn_split_combine_kernel(const AttnArgs A, const float* __restrict__ ws, int n_splits, int n_tok, int dvp,
                          const float* __restrict__ rot_tab) {
  extern __shared__ float res[];   // [H][dv]
  const int n = blockIdx.x, H = A.H, dv = A.dv, stride = dvp + 2;
  for (int e = threadIdx.x; e < H * dv; e += blockDim.x) {
    const int h = e / dv, c = e - h * dv;
    float M = A.sink ? A.sink[h] : -INFINITY;
    for (int sp = 0; sp < n_splits; ++sp) M = fmaxf(M, ws[((static_cast<int64_t>(sp) * n_tok + n) * H + h) * stride]);
    float L = A.sink ? expf(A.sink[h] - M) : 0.f, O = 0.f;
    for (int sp = 0; sp < n_splits; ++sp) {
      const float* src = ws + ((static_cast<int64_t>(sp) * n_tok + n) * H + h) * stride;
      const float f = src[0] == -INFINITY ? 0.f : expf(src[0] - M);
      L = fmaf(src[1], f, L);
      O = fmaf(src[2 + c], f, O);
    }
    res[e] = O / L;
  }
  __syncthreads();
  T* out = static_cast<T*>(A.out) + static_cast<int64_t>(n) * A.out_tok_stride;
  const T* gate = static_cast<const T*>(A.gate);
  if (A.unrotate) {
    const int vh = dv / 2;
    for (int e = threadIdx.x; e < H * vh; e += blockDim.x) {
      const int h = e / vh, i = e - h * vh;
      const float cf = rot_tab[(static_cast<int64_t>(n) * vh + i) * 2], sf = rot_tab[(static_cast<int64_t>(n) * vh + i) * 2 + 1];
      const int a = A.interleaved ? 2 * i : i, b = A.interleaved ? 2 * i + 1 : i + vh;
      const float u = res[h * dv + a], w = res[h * dv + b];
      float ya = u * cf + w * sf, yb = w * cf - u * sf;
      if (gate) {
        const float gt = sigmoid_(Cvt<T>::to_f32(gate[static_cast<int64_t>(n) * A.gate_stride + h]));
        ya *= gt;
        yb *= gt;
      }
      out[h * A.out_head_stride + a] = Cvt<T>::from_f32(ya);
      out[h * A.out_head_stride + b] = Cvt<T>::from_f32(yb);
    }
    if (dv & 1)
      for (int h = threadIdx.x; h < H; h += blockDim.x)
        out[h * A.out_head_stride + dv - 1] = Cvt<T>::from_f32(res[h * dv + dv - 1]);
  } else {
    for (int e = threadIdx.x; e < H * dv; e += blockDim.x) {
      const int h = e / dv, c = e - h * dv;
      float y = res[e];
      if (gate) y *= sigmoid_(Cvt<T>::to_f32(gate[static_cast<int64_t>(n) * A.gate_stride + h]));
      if (A.out_f32) static_cast<float*>(A.out)[static_cast<int64_t>(n) * A.out_tok_stride + h * A.out_head_stride + c] = y;
      else out[h * A.out_head_stride + c] = Cvt<T>::from_f32(y);
    }
  }
}

struct TcPlan {
  int dv8, hw, stages;
  size_t smem;
};

inline bool tc_plan(int H, int G, int dk, int dv, bool has_talk, bool same_pool, bool unrotate, int dtype, TcPlan* plan,
                    bool stage_q = false) {
  if (dtype == B200_DTYPE_F32 || dk % 16 || dv % 8 || dv > 256 || H % G) return false;
  const int dv8 = dv <= 64 ? 8 : (dv <= 128 ? 16 : 32), dvp = dv8 * 8;
  // two heads per warp pay when the CTA's heads share what is staged: with a mixing matrix (all heads' raw scores are
  // formed anyway) or when one kv head serves more heads than a CTA has warps; plain grouped-query layouts run one
  // head per warp, which halves the staged kv heads per CTA and lets two CTAs share an SM
  const int hw = (dv8 <= 16 && H > kTcWarps && (has_talk || H / G > kTcWarps)) ? 2 : 1;
  const int gs = has_talk ? G : std::min(G, (kTcWarps * hw + H / G - 1) / (H / G) + 1);
  const bool alias = same_pool && dvp <= dk;
  size_t stage = static_cast<size_t>(gs) * kTcKeys * (dk + 8) * 2;
  if (!alias) stage += static_cast<size_t>(gs) * kTcKeys * (dvp + 8) * 2;
  size_t rest = 0;
  if (has_talk) rest = sizeof(float) * (static_cast<size_t>(H) * kTcRows * kTcRawStride + static_cast<size_t>(kTcWarps) * hw * H);
  if (stage_q) rest += static_cast<size_t>(kTcWarps) * hw * kTcRows * (dk + 8) * 2;   // the staged query rows
  const size_t slab = unrotate ? sizeof(float) * kTcWarps * kTcRows * static_cast<size_t>(dvp) : 0;
  const size_t cap = 227 * 1024;
  int stages = 2;
  if (std::max(2 * stage + rest, slab) > cap) stages = 1;
  const size_t bytes = std::max(stages * stage + rest, slab);
  if (bytes > cap) return false;
  if (plan) *plan = TcPlan{dv8, hw, stages, bytes};
  return true;
}

// ---- short causal convolution + SiLU -----------------------------------------------------------------------------
struct SeqSpan {
  int tok0;   // first packed row
  int count;  // tokens in this step
  int slot;   // state slot
  int fresh;  // 1: the sequence starts here (state is zero)
};

constexpr int kConvTokens = 64;   // tokens per CTA; at least taps - 1, so only a sequence's first CTA reads the carried inputs

template <typename T>
__global__ void __launch_bounds__(128)
causal_conv_silu_kernel(T* __restrict__ out, int64_t out_stride, const T* __restrict__ x, int64_t x_stride,
                        const T* __restrict__ w, float* __restrict__ tail, const SeqSpan* __restrict__ seqs, int C,
                        int taps) {
  const SeqSpan sq = seqs[blockIdx.x];
  const int t0 = blockIdx.y * kConvTokens;
  if (t0 >= sq.count) return;
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  if (c >= C) return;
  constexpr int kMaxTaps = 8;
  float wr[kMaxTaps], old[kMaxTaps];
#pragma unroll
  for (int i = 0; i < kMaxTaps; ++i) {
    wr[i] = i < taps ? Cvt<T>::to_f32(w[static_cast<int64_t>(c) * taps + i]) : 0.f;
    old[i] = 0.f;
  }
  float* tl = tail + static_cast<int64_t>(sq.slot) * (taps - 1) * C + c;   // [taps - 1][C], oldest first
  if (t0 == 0 && !sq.fresh)
#pragma unroll
    for (int i = 0; i < kMaxTaps - 1; ++i)
      if (i < taps - 1) old[i] = tl[static_cast<int64_t>(i) * C];
  const T* xc = x + static_cast<int64_t>(sq.tok0) * x_stride + c;
  auto input = [&](int t) -> float {    // the channel's input at step t of this portion; t < 0 reaches into the carry
    if (t >= 0) return Cvt<T>::to_f32(xc[static_cast<int64_t>(t) * x_stride]);
    float r = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxTaps - 1; ++i)
      if (i == taps - 1 + t) r = old[i];
    return r;
  };
  const int t1 = min(sq.count, t0 + kConvTokens);
  for (int t = t0; t < t1; ++t) {
    float y = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i)
      if (i < taps) y = fmaf(wr[i], input(t - (taps - 1 - i)), y);
    out[static_cast<int64_t>(sq.tok0 + t) * out_stride + c] = Cvt<T>::from_f32(y * sigmoid_(y));
  }
  if (t0 == 0) {
    // the new carry: the portion's last taps - 1 inputs (older ones come from the old carry when the portion is short)
    float nw[kMaxTaps];
#pragma unroll
    for (int i = 0; i < kMaxTaps - 1; ++i) nw[i] = (i < taps - 1) ? input(sq.count - (taps - 1) + i) : 0.f;
#pragma unroll
    for (int i = 0; i < kMaxTaps - 1; ++i)
      if (i < taps - 1) tl[static_cast<int64_t>(i) * C] = nw[i];
  }
}

// ---- gated delta rule --------------------------------------------------------------------------------------------
// One CTA per (sequence, head, 32 value columns): a value column's part of the state never meets another column's, so
// columns are independent.  Four adjacent lanes share a column; lane r keeps the state rows i = r, r + 4, ... of that
// column in registers for the whole portion.  Eight tokens (fewer for the widest keys) are staged at a time, double buffered (the raw loads of
// the next eight are issued before the current eight are computed): their activated q and k (unit length per head, q
// also scaled), the decays g = exp(-exp(A_log) softplus(a + dt_bias)), the write strength sigmoid(b) and the CTA's
// value columns.  Per token: S <- g S and d = S^T k in one pass, u = beta (v - d), then S <- S + k u and
// o = S^T q in a second pass; the four lanes' partial sums meet in two shuffles.
constexpr int kDeltaNT = 128;
constexpr int kDeltaCols = kDeltaNT / 4;

struct DeltaArgs {
  float* o_raw;
  const void* q; const void* k; const void* v; int64_t in_stride;
  const void* beta; int64_t beta_stride;
  const void* a; int64_t a_stride;
  const void* dt_bias; const void* a_log;
  float* state; const SeqSpan* seqs;
  int H, G, dk, dv; float unit_eps, q_scale;
};

__host__ __device__ constexpr int delta_chunk(int dk_padded) { return dk_padded >= 256 ? 2 : (dk_padded >= 128 ? 4 : 8); }

template <typename T, int DK>
__global__ void __launch_bounds__(kDeltaNT)
delta_scan_kernel(const DeltaArgs A) {
  extern __shared__ __align__(16) float smem[];
  constexpr int RW4 = DK / 4;
  constexpr int kDeltaChunk = delta_chunk(DK);
  constexpr int row_len = 3 * DK + kDeltaCols + 4;      // q | k | g (each grouped by r) | v[32] | beta, pad
  constexpr int kPer = (kDeltaChunk * row_len + kDeltaNT - 1) / kDeltaNT;   // staged elements per thread and chunk
  const SeqSpan sq = A.seqs[blockIdx.x];
  const int h = blockIdx.y, H = A.H, dk = A.dk, dv = A.dv;
  const int gq = h / (H / A.G);                          // the q / k head this value head reads
  const int r = threadIdx.x & 3, cl = threadIdx.x >> 2;
  const int col0 = blockIdx.z * kDeltaCols, col = col0 + cl;
  const int ncol = min(kDeltaCols, dv - col0);
  const bool has_col = col < dv;
  float* st = A.state + (static_cast<int64_t>(sq.slot) * H + h) * dk * dv;
  float S[RW4];
#pragma unroll
  for (int kk = 0; kk < RW4; ++kk) {
    const int i = 4 * kk + r;
    S[kk] = (!sq.fresh && i < dk && has_col) ? st[static_cast<int64_t>(i) * dv + col] : 0.f;
  }
  const T* qp = static_cast<const T*>(A.q);
  const T* kp = static_cast<const T*>(A.k);
  const T* vp = static_cast<const T*>(A.v);
  const T* bp = static_cast<const T*>(A.beta);
  const T* ap = static_cast<const T*>(A.a);
  const T* dtb = static_cast<const T*>(A.dt_bias);
  const float a_rate = expf(Cvt<T>::to_f32(static_cast<const T*>(A.a_log)[h]));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* buf0 = smem;
  float* buf1 = smem + kDeltaChunk * row_len;
  T rawv[kPer];
  // staged element e of a chunk: token e / row_len, slot e % row_len; slot r * RW4 + kk of a section holds row 4 kk + r.
  // `fetch` only issues the loads (nothing waits for them until `commit`), so they fly while a chunk is computed.
  auto fetch = [&](int t0) {
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int e = threadIdx.x + u * kDeltaNT;
      const int tt = e / row_len, sl = e - tt * row_len;
      rawv[u] = Cvt<T>::from_f32(0.f);
      if (tt < kDeltaChunk && t0 + tt < sq.count) {
        const int64_t tok = sq.tok0 + t0 + tt;
        if (sl < 3 * DK) {
          const int which = sl / DK, s2 = sl - which * DK;
          const int i = 4 * (s2 % RW4) + s2 / RW4;
          if (i < dk) {
            if (which == 0) rawv[u] = qp[tok * A.in_stride + gq * dk + i];
            else if (which == 1) rawv[u] = kp[tok * A.in_stride + gq * dk + i];
            else rawv[u] = ap[tok * A.a_stride + h * dk + i];
          }
        } else if (sl < 3 * DK + kDeltaCols) {
          if (sl - 3 * DK < ncol) rawv[u] = vp[tok * A.in_stride + h * dv + col0 + sl - 3 * DK];
        } else if (sl == 3 * DK + kDeltaCols) {
          rawv[u] = bp[tok * A.beta_stride + h];
        }
      }
    }
  };
  auto commit = [&](float* dst, int n_valid) {
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int e = threadIdx.x + u * kDeltaNT;
      const int tt = e / row_len, sl = e - tt * row_len;
      if (tt < n_valid) {
        float val = Cvt<T>::to_f32(rawv[u]);
        if (sl >= 2 * DK && sl < 3 * DK) {
          const int s2 = sl - 2 * DK;
          const int i = 4 * (s2 % RW4) + s2 / RW4;
          val = i < dk ? expf(-a_rate * softplus_(val + Cvt<T>::to_f32(dtb[h * dk + i]))) : 0.f;
        } else if (sl == 3 * DK + kDeltaCols) {
          val = sigmoid_(val);
        }
        dst[e] = val;
      }
    }
  };
  auto unit = [&](float* dst, int n_valid) {   // warp w brings tokens w, w + 4, ... to unit length per head
    for (int tt = warp; tt < n_valid; tt += kDeltaNT / 32) {
      float* row = dst + tt * row_len;
      float sq2 = 0.f, sk2 = 0.f;
      for (int i = lane; i < DK; i += 32) {
        sq2 = fmaf(row[i], row[i], sq2);
        sk2 = fmaf(row[DK + i], row[DK + i], sk2);
      }
      const float iq = rsqrtf(warp_sum(sq2) + A.unit_eps) * A.q_scale;
      const float ik = rsqrtf(warp_sum(sk2) + A.unit_eps);
      for (int i = lane; i < DK; i += 32) {
        row[i] *= iq;
        row[DK + i] *= ik;
      }
    }
  };
  fetch(0);
  commit(buf0, min(kDeltaChunk, sq.count));
  __syncthreads();
  unit(buf0, min(kDeltaChunk, sq.count));
  __syncthreads();
  for (int t0 = 0; t0 < sq.count; t0 += kDeltaChunk) {
    const float* cur = ((t0 / kDeltaChunk) & 1) ? buf1 : buf0;
    float* nxt = ((t0 / kDeltaChunk) & 1) ? buf0 : buf1;
    const int n_here = min(kDeltaChunk, sq.count - t0);
    const int n_next = min(kDeltaChunk, sq.count - t0 - kDeltaChunk);
    if (n_next > 0) fetch(t0 + kDeltaChunk);
    for (int tt = 0; tt < n_here; ++tt) {
      const float* row = cur + tt * row_len;
      const float* qr = row + r * RW4;
      const float* kr = row + DK + r * RW4;
      const float* gr = row + 2 * DK + r * RW4;
      const float vc = row[3 * DK + cl], beta = row[3 * DK + kDeltaCols];
      float d0 = 0.f, d1 = 0.f;
#pragma unroll
      for (int kk = 0; kk < RW4; kk += 4) {
        const float4 g4 = *reinterpret_cast<const float4*>(gr + kk);
        const float4 k4 = *reinterpret_cast<const float4*>(kr + kk);
        S[kk] *= g4.x;
        d0 = fmaf(S[kk], k4.x, d0);
        S[kk + 1] *= g4.y;
        d1 = fmaf(S[kk + 1], k4.y, d1);
        S[kk + 2] *= g4.z;
        d0 = fmaf(S[kk + 2], k4.z, d0);
        S[kk + 3] *= g4.w;
        d1 = fmaf(S[kk + 3], k4.w, d1);
      }
      float d = d0 + d1;
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      const float u = beta * (vc - d);
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int kk = 0; kk < RW4; kk += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kr + kk);
        const float4 q4 = *reinterpret_cast<const float4*>(qr + kk);
        S[kk] = fmaf(k4.x, u, S[kk]);
        o0 = fmaf(S[kk], q4.x, o0);
        S[kk + 1] = fmaf(k4.y, u, S[kk + 1]);
        o1 = fmaf(S[kk + 1], q4.y, o1);
        S[kk + 2] = fmaf(k4.z, u, S[kk + 2]);
        o0 = fmaf(S[kk + 2], q4.z, o0);
        S[kk + 3] = fmaf(k4.w, u, S[kk + 3]);
        o1 = fmaf(S[kk + 3], q4.w, o1);
      }
      float o = o0 + o1;
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (r == 0 && has_col) A.o_raw[(static_cast<int64_t>(sq.tok0 + t0 + tt) * H + h) * dv + col] = o;
    }
    if (n_next > 0) {
      commit(nxt, n_next);       // `nxt` was last read two chunks ago, before the barrier that ended that chunk
      __syncthreads();
      unit(nxt, n_next);
    }
    __syncthreads();
  }
#pragma unroll
  for (int kk = 0; kk < RW4; ++kk) {
    const int i = 4 * kk + r;
    if (i < dk && has_col) st[static_cast<int64_t>(i) * dv + col] = S[kk];
  }
}

// ---- o * rsqrt(mean(o^2) + eps) * w * sigmoid(gate); one warp per (token, head) ------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
head_rmsnorm_gated_kernel(T* __restrict__ out, const float* __restrict__ x, const T* __restrict__ w,
                          const T* __restrict__ gate, int64_t gate_stride, float eps, int64_t rows, int H, int dv) {
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
  for (int i = lane; i < dv; i += 32) {
    float y = xr[i] * inv * Cvt<T>::to_f32(w[i]);
    if (gr) y *= sigmoid_(Cvt<T>::to_f32(gr[i]));
    out[row * dv + i] = Cvt<T>::from_f32(y);
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_rms_norm(void* out, int64_t out_stride, const void* x, int64_t x_stride, int x_is_f32, const void* weight,
                  float weight_offset, float eps, int rows, int width, int dtype, void* stream) {
  if (rows < 0 || width <= 0) return fail(B200_EINVAL, "b200_rms_norm: bad sizes");
  if (rows == 0) return 0;
  if (!out || !x || !weight) return fail(B200_EINVAL, "b200_rms_norm: null pointer");
  return hybrid_by_dtype(dtype, "b200_rms_norm", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto s = static_cast<cudaStream_t>(stream);
    if (x_is_f32)
      rms_norm_kernel<T, float><<<rows, 256, 0, s>>>(static_cast<T*>(out), out_stride, static_cast<const float*>(x),
                                                     x_stride, static_cast<const T*>(weight), weight_offset, eps, width);
    else
      rms_norm_kernel<T, T><<<rows, 256, 0, s>>>(static_cast<T*>(out), out_stride, static_cast<const T*>(x), x_stride,
                                                 static_cast<const T*>(weight), weight_offset, eps, width);
    return check_launch("b200_rms_norm");
  });
}

int b200_residual_add2_norm(float* x, const void* a, int64_t a_stride, const void* b, int64_t b_stride, const void* w_next,
                            float weight_offset, void* out_next, float eps, int rows, int width, int dtype, void* stream) {
  if (rows < 0 || width <= 0 || width > 40000) return fail(B200_EINVAL, "b200_residual_add2_norm: bad sizes");
  if (rows == 0) return 0;
  if (!x || !a || (w_next && !out_next)) return fail(B200_EINVAL, "b200_residual_add2_norm: null pointer");
  const size_t smem = static_cast<size_t>(width) * sizeof(float);
  return hybrid_by_dtype(dtype, "b200_residual_add2_norm", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto kern = residual_add2_norm_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<rows, 256, smem, static_cast<cudaStream_t>(stream)>>>(x, static_cast<const T*>(a), a_stride,
                                                                static_cast<const T*>(b), b_stride,
                                                                static_cast<const T*>(w_next), weight_offset,
                                                                static_cast<T*>(out_next), eps, width);
    return check_launch("b200_residual_add2_norm");
  });
}

int b200_xielu(void* out, const void* z, int64_t z_stride, const void* pq, int rows, int ff, int dtype, void* stream) {
  if (rows < 0 || ff <= 0) return fail(B200_EINVAL, "b200_xielu: bad sizes");
  if (rows == 0) return 0;
  if (!out || !z || !pq) return fail(B200_EINVAL, "b200_xielu: null pointer");
  const int es = dtype_size(dtype);
  const bool vec = es > 0 && (ff * es) % 16 == 0 && (z_stride * es) % 16 == 0 && aligned16(z) && aligned16(out);
  const int per = vec ? 256 * (16 / es) : 256;
  const dim3 grid(std::min((ff + per - 1) / per, 64), rows);
  return hybrid_by_dtype(dtype, "b200_xielu", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    xielu_kernel<T><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<T*>(out), static_cast<const T*>(z),
                                                                         z_stride, static_cast<const T*>(pq), ff, vec);
    return check_launch("b200_xielu");
  });
}

int b200_rotary_kv_append(void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v, int64_t v_stride,
                          void* k_pool, void* v_pool, const int64_t* slot_mapping, const int32_t* tok_pos, int n_tok, int H,
                          int G, int dk, int dv, int rot_dims, float rot_base, int rotate_values, int interleaved,
                          int block_size, int64_t max_blocks, float* value_rot, int dtype, void* stream) {
  if (n_tok < 0 || H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || block_size <= 0 || max_blocks <= 0)
    return fail(B200_EINVAL, "b200_rotary_kv_append: bad sizes");
  if (rot_dims < 0 || rot_dims > dk || (rot_dims & 1)) return fail(B200_ESHAPE, "b200_rotary_kv_append: rot_dims %d", rot_dims);
  if (n_tok == 0) return 0;
  if (!q || !k || !v || !k_pool || !v_pool || !slot_mapping || !tok_pos) return fail(B200_EINVAL, "b200_rotary_kv_append: null pointer");
  const size_t smem = sizeof(float) * (static_cast<size_t>(rot_dims) + (rotate_values ? dv : 0) + 4);
  return hybrid_by_dtype(dtype, "b200_rotary_kv_append", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    rotary_kv_append_kernel<T><<<n_tok, 256, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(q), q_stride, static_cast<const T*>(k), k_stride, static_cast<const T*>(v), v_stride,
        static_cast<T*>(k_pool), static_cast<T*>(v_pool), slot_mapping, tok_pos, H, G, dk, dv, rot_dims,
        static_cast<double>(rot_base), rotate_values, interleaved, block_size, rotate_values ? value_rot : nullptr);
    return check_launch("b200_rotary_kv_append");
  });
}

int b200_norm_append(const void* x, int64_t x_stride, const void* weight, float weight_offset, float eps, void* pool,
                     const int64_t* slot_mapping, int n_tok, int width, int dtype, void* stream) {
  if (n_tok < 0 || width <= 0) return fail(B200_EINVAL, "b200_norm_append: bad sizes");
  if (n_tok == 0) return 0;
  if (!x || !weight || !pool || !slot_mapping) return fail(B200_EINVAL, "b200_norm_append: null pointer");
  return hybrid_by_dtype(dtype, "b200_norm_append", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    norm_append_kernel<T><<<n_tok, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const T*>(x), x_stride, static_cast<const T*>(weight), weight_offset, eps, static_cast<T*>(pool),
        slot_mapping, width);
    return check_launch("b200_norm_append");
  });
}

int b200_mixed_paged_attn(void* out, int64_t out_tok_stride, int64_t out_head_stride, const void* q, int64_t q_tok_stride,
                          int64_t q_head_stride, const void* gate, int64_t gate_stride, const void* k_pool,
                          const void* v_pool, const int32_t* block_tables, int table_stride, const int32_t* tok_row,
                          const int32_t* tok_pos, int n_tok, const float* talk, const float* sink, float scale,
                          float softcap, int window, int keep_first, int unrotate, int interleaved, float rot_base, int H,
                          int G, int dk, int dv, int block_size, int dtype, void* stream) {
  return b200_mixed_paged_attn_ext(out, out_tok_stride, out_head_stride, q, q_tok_stride, q_head_stride, gate, gate_stride,
                                   k_pool, v_pool, block_tables, table_stride, tok_row, tok_pos, n_tok, talk, sink, scale,
                                   softcap, window, keep_first, 0, unrotate, interleaved, rot_base, H, G, dk, dv, dv, 1, 0,
                                   block_size, dtype, stream);
}

int b200_mixed_paged_attn_ext(void* out, int64_t out_tok_stride, int64_t out_head_stride, const void* q,
                              int64_t q_tok_stride, int64_t q_head_stride, const void* gate, int64_t gate_stride,
                              const void* k_pool, const void* v_pool, const int32_t* block_tables, int table_stride,
                              const int32_t* tok_row, const int32_t* tok_pos, int n_tok, const float* talk,
                              const float* sink, float scale, float softcap, int window, int keep_first, int chunk,
                              int unrotate, int interleaved, float rot_base, int H, int G, int dk, int dv, int v_row,
                              int v_div, int out_f32, int block_size, int dtype, void* stream) {
  if (out_f32 && unrotate) return fail(B200_EINVAL, "b200_mixed_paged_attn: fp32 outputs are not turned back");
  if (n_tok < 0 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || block_size <= 0 || chunk < 0 || v_row < dv ||
      v_div < 1 || G % v_div)
    return fail(B200_EINVAL, "b200_mixed_paged_attn: bad sizes");
  if (dv > 512) return fail(B200_ESHAPE, "b200_mixed_paged_attn: value size %d beyond 512", dv);
  if (n_tok == 0) return 0;
  if (!out || !q || !k_pool || !v_pool || !block_tables || !tok_row || !tok_pos)
    return fail(B200_EINVAL, "b200_mixed_paged_attn: null pointer");
  AttnArgs A{out, out_tok_stride, out_head_stride, q, q_tok_stride, q_head_stride, gate, gate_stride, k_pool, v_pool,
             block_tables, table_stride, tok_row, tok_pos, talk, sink, scale, window, keep_first, unrotate, interleaved,
             static_cast<double>(rot_base), H, G, dk, dv, block_size, softcap, chunk, v_row, v_div, 0, out_f32};
  const int dvc = dv <= 64 ? 2 : (dv <= 128 ? 4 : (dv <= 256 ? 8 : 16));
  const int hp = dvc <= 4 ? 8 : (dvc == 8 ? 4 : 2);
  const int nhs = talk ? H : std::min(hp, H);
  // the score staging area [warps][nhs][32] is reused for the [hp][dv] results: give it room for both
  const size_t raw = std::max<size_t>(static_cast<size_t>(kAttnWarpsRow) * nhs * 32, static_cast<size_t>(hp) * dv);
  const size_t smem = sizeof(float) * (static_cast<size_t>(nhs) * dk + raw + (talk ? static_cast<size_t>(hp) * H : 0) +
                                       static_cast<size_t>(kAttnWarpsRow) * hp * (dv + 2));
  if (smem > 200 * 1024) return fail(B200_ESHAPE, "b200_mixed_paged_attn: %zu bytes of shared memory", smem);
  const dim3 grid(n_tok, (H + hp - 1) / hp);
  return hybrid_by_dtype(dtype, "b200_mixed_paged_attn", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto launch = [&](auto kern) {
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      kern<<<grid, kAttnWarpsRow * 32, smem, static_cast<cudaStream_t>(stream)>>>(A);
    };
    if (dvc == 2) launch(mixed_paged_attn_kernel<T, 8, 2>);
    else if (dvc == 4) launch(mixed_paged_attn_kernel<T, 8, 4>);
    else if (dvc == 8) launch(mixed_paged_attn_kernel<T, 4, 8>);
    else launch(mixed_paged_attn_kernel<T, 2, 16>);
    return check_launch("b200_mixed_paged_attn");
  });
}

int b200_mixed_prompt_attn_supported(int H, int G, int dk, int dv, int has_talk, int same_pool, int unrotate, int dtype) {
  if (H <= 0 || G <= 0) return 0;
  return tc_plan(H, G, dk, dv, has_talk != 0, same_pool != 0, unrotate != 0, dtype, nullptr) ? 1 : 0;
}

int b200_mixed_prompt_attn_splits(int n_tiles, int key_tiles, int H, int G, int dk, int dv, int has_talk, int same_pool,
                                  int unrotate, int dtype) {
  TcPlan plan;
  if (n_tiles <= 0 || H <= 0 || G <= 0 || !tc_plan(H, G, dk, dv, has_talk != 0, same_pool != 0, unrotate != 0, dtype, &plan))
    return 1;
  const int ctas = n_tiles * ((H + kTcWarps * plan.hw - 1) / (kTcWarps * plan.hw));
  if (ctas >= kNumSMs) return 1;
  return std::max(1, std::min({8, (2 * kNumSMs + ctas - 1) / ctas, key_tiles / 4}));
}

size_t b200_mixed_prompt_attn_workspace(int n_splits, int n_tok, int H, int dv) {
  if (n_splits <= 1 || n_tok <= 0 || H <= 0 || dv <= 0) return 0;
  const int dvp = (dv <= 64 ? 8 : (dv <= 128 ? 16 : 32)) * 8;
  return sizeof(float) * static_cast<size_t>(n_splits) * n_tok * H * (dvp + 2);
}

int b200_mixed_prompt_attn(void* out, int64_t out_tok_stride, int64_t out_head_stride, const void* q, int64_t q_tok_stride,
                           int64_t q_head_stride, const void* gate, int64_t gate_stride, const void* k_pool,
                           const void* v_pool, const int32_t* block_tables, int table_stride, const int32_t* tiles,
                           int n_tiles, const int32_t* tok_pos, int n_tok, const float* talk, const float* sink,
                           float scale, float softcap, int window, int keep_first, const float* value_rot, int interleaved,
                           int H, int G, int dk, int dv, int block_size, int n_splits, float* workspace, int dtype,
                           void* stream) {
  return b200_mixed_prompt_attn_ext(out, out_tok_stride, out_head_stride, q, q_tok_stride, q_head_stride, gate, gate_stride,
                                    k_pool, v_pool, block_tables, table_stride, tiles, n_tiles, tok_pos, n_tok, talk, sink,
                                    scale, softcap, window, keep_first, 0, value_rot, interleaved, H, G, dk, dv, dv, 1, 0, 0,
                                    block_size, n_splits, workspace, dtype, stream);
}

int b200_mixed_prompt_attn_ext(void* out, int64_t out_tok_stride, int64_t out_head_stride, const void* q,
                               int64_t q_tok_stride, int64_t q_head_stride, const void* gate, int64_t gate_stride,
                               const void* k_pool, const void* v_pool, const int32_t* block_tables, int table_stride,
                               const int32_t* tiles, int n_tiles, const int32_t* tok_pos, int n_tok, const float* talk,
                               const float* sink, float scale, float softcap, int window, int keep_first, int chunk,
                               const float* value_rot, int interleaved, int H, int G, int dk, int dv, int v_row, int v_div,
                               int heads_as_rows, int out_f32, int block_size, int n_splits, float* workspace, int dtype,
                               void* stream) {
  if (out_f32 && value_rot) return fail(B200_EINVAL, "b200_mixed_prompt_attn: fp32 outputs are not turned back");
  if (chunk < 0 || v_row < dv || v_row % 8 || v_div < 1 || G % v_div)
    return fail(B200_EINVAL, "b200_mixed_prompt_attn: bad mask or value layout");
  if (heads_as_rows && (G != 1 || talk || gate || value_rot))
    return fail(B200_EINVAL, "b200_mixed_prompt_attn: heads as rows need one kv head and no mixing, gate or value rotation");
  if (heads_as_rows && (!aligned16(q) || ((q_tok_stride | q_head_stride) & 7)))
    return fail(B200_ESHAPE, "b200_mixed_prompt_attn: heads as rows need 16-byte aligned query rows");
  const int H_real = H;
  if (heads_as_rows) H = (H + 15) / 16;      // the kernel's heads are groups of 16 rows
  if (n_tiles < 0 || n_tok < 0 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || block_size <= 0 || n_splits < 1 ||
      n_splits > 64)
    return fail(B200_EINVAL, "b200_mixed_prompt_attn: bad sizes");
  if (n_tiles == 0) return 0;
  if (!out || !q || !k_pool || !v_pool || !block_tables || !tiles || !tok_pos || (n_splits > 1 && !workspace))
    return fail(B200_EINVAL, "b200_mixed_prompt_attn: null pointer");
  if ((q_tok_stride | q_head_stride | out_tok_stride | out_head_stride) & 1)
    return fail(B200_ESHAPE, "b200_mixed_prompt_attn: odd strides");
  TcPlan plan;
  // query rows are staged where few warps are resident anyway: heads on the rows, and the widest value layout (one CTA
  // per SM by its registers) when its rows allow 16-byte reads
  const bool q_ok = aligned16(q) && !((q_tok_stride | q_head_stride) & 7);
  const bool ext_call = chunk > 0 || v_div > 1 || v_row != dv || heads_as_rows || out_f32;
  bool stage_q = heads_as_rows || (ext_call && dv > 128 && q_ok);
  if (stage_q && !heads_as_rows && !tc_plan(H, G, dk, dv, talk != nullptr, k_pool == v_pool, value_rot != nullptr, dtype, &plan, true))
    stage_q = false;
  if (!tc_plan(H, G, dk, dv, talk != nullptr, k_pool == v_pool, value_rot != nullptr, dtype, &plan, stage_q))
    return fail(B200_ESHAPE, "b200_mixed_prompt_attn: sizes off the tensor-core grid (dk %d, dv %d)", dk, dv);
  AttnArgs A{out, out_tok_stride, out_head_stride, q, q_tok_stride, q_head_stride, gate, gate_stride, k_pool, v_pool,
             block_tables, table_stride, nullptr, tok_pos, talk, sink, scale, window, keep_first, value_rot != nullptr,
             interleaved, 0.0, H, G, dk, dv, block_size, softcap, chunk, v_row, v_div, heads_as_rows ? H_real : 0,
             out_f32, stage_q ? 1 : 0};
  const dim3 grid(n_tiles, (H + kTcWarps * plan.hw - 1) / (kTcWarps * plan.hw), n_splits);
  return hybrid_by_dtype(dtype, "b200_mixed_prompt_attn", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    if constexpr (std::is_same_v<T, float>) {
      return fail(B200_ESHAPE, "b200_mixed_prompt_attn: 16-bit storage types only");
    } else {
      auto s = static_cast<cudaStream_t>(stream);
      auto launch = [&](auto kern) {
        if (plan.smem > 48 * 1024)
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smem));
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        kern<<<grid, kTcWarps * 32, plan.smem, s>>>(A, tiles, value_rot, workspace, n_tok, plan.stages);
      };
      const bool ext = ext_call;
      if (ext) {
        if (plan.dv8 == 8 && plan.hw == 1) launch(mixed_prompt_attn_kernel<T, 8, 1, true>);
        else if (plan.dv8 == 8) launch(mixed_prompt_attn_kernel<T, 8, 2, true>);
        else if (plan.dv8 == 16 && plan.hw == 1) launch(mixed_prompt_attn_kernel<T, 16, 1, true>);
        else if (plan.dv8 == 16) launch(mixed_prompt_attn_kernel<T, 16, 2, true>);
        else launch(mixed_prompt_attn_kernel<T, 32, 1, true>);
      } else {
        if (plan.dv8 == 8 && plan.hw == 1) launch(mixed_prompt_attn_kernel<T, 8, 1, false>);
        else if (plan.dv8 == 8) launch(mixed_prompt_attn_kernel<T, 8, 2, false>);
        else if (plan.dv8 == 16 && plan.hw == 1) launch(mixed_prompt_attn_kernel<T, 16, 1, false>);
        else if (plan.dv8 == 16) launch(mixed_prompt_attn_kernel<T, 16, 2, false>);
        else launch(mixed_prompt_attn_kernel<T, 32, 1, false>);
      }
      int rc = check_launch("b200_mixed_prompt_attn");
      if (rc != 0 || n_splits == 1) return rc;
      // every packed row belongs to exactly one tile, so the merge runs over all rows
      A.H = H_real;
      const size_t smem_c = sizeof(float) * static_cast<size_t>(H_real) * dv;
      auto comb = attn_split_combine_kernel<T>;
      if (smem_c > 48 * 1024) cudaFuncSetAttribute(comb, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_c));
      comb<<<n_tok, 256, smem_c, s>>>(A, workspace, n_splits, n_tok, plan.dv8 * 8, value_rot);
      return check_launch("b200_mixed_prompt_attn (merge)");
    }
  });
}

int b200_causal_conv_silu(void* out, int64_t out_stride, const void* x, int64_t x_stride, const void* w, float* tail,
                          const int32_t* seqs, int n_seqs, int max_count, int C, int taps, int dtype, void* stream) {
  if (n_seqs < 0 || C <= 0 || taps < 1 || max_count < 0) return fail(B200_EINVAL, "b200_causal_conv_silu: bad sizes");
  if (taps > 8) return fail(B200_ESHAPE, "b200_causal_conv_silu: %d taps beyond 8", taps);
  if (n_seqs == 0 || max_count == 0) return 0;
  if (!out || !x || !w || !seqs || (taps > 1 && !tail)) return fail(B200_EINVAL, "b200_causal_conv_silu: null pointer");
  const dim3 grid(n_seqs, (max_count + kConvTokens - 1) / kConvTokens, (C + 127) / 128);
  return hybrid_by_dtype(dtype, "b200_causal_conv_silu", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    causal_conv_silu_kernel<T><<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(out), out_stride, static_cast<const T*>(x), x_stride, static_cast<const T*>(w), tail,
        reinterpret_cast<const SeqSpan*>(seqs), C, taps);
    return check_launch("b200_causal_conv_silu");
  });
}

int b200_delta_scan(float* o_raw, const void* q, const void* k, const void* v, int64_t in_stride, const void* beta_logit,
                    int64_t beta_stride, const void* a_logit, int64_t a_stride, const void* dt_bias, const void* a_log,
                    float* state, const int32_t* seqs, int n_seqs, int H, int G, int dk, int dv, float unit_eps,
                    float q_scale, int dtype, void* stream) {
  if (n_seqs < 0 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0) return fail(B200_EINVAL, "b200_delta_scan: bad sizes");
  if (dk > 256) return fail(B200_ESHAPE, "b200_delta_scan: key size %d beyond 256", dk);
  if (n_seqs == 0) return 0;
  if (!o_raw || !q || !k || !v || !beta_logit || !a_logit || !dt_bias || !a_log || !state || !seqs)
    return fail(B200_EINVAL, "b200_delta_scan: null pointer");
  const int dkt = dk <= 32 ? 32 : (dk <= 64 ? 64 : (dk <= 128 ? 128 : 256));
  const size_t smem = sizeof(float) * 2 * delta_chunk(dkt) * (3 * static_cast<size_t>(dkt) + kDeltaCols + 4);
  const dim3 grid(n_seqs, H, (dv + kDeltaCols - 1) / kDeltaCols);
  DeltaArgs A{o_raw, q, k, v, in_stride, beta_logit, beta_stride, a_logit, a_stride, dt_bias, a_log, state,
              reinterpret_cast<const SeqSpan*>(seqs), H, G, dk, dv, unit_eps, q_scale};
  return hybrid_by_dtype(dtype, "b200_delta_scan", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto s = static_cast<cudaStream_t>(stream);
    auto launch = [&](auto kern) {
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      kern<<<grid, kDeltaNT, smem, s>>>(A);
    };
    if (dkt == 32) launch(delta_scan_kernel<T, 32>);
    else if (dkt == 64) launch(delta_scan_kernel<T, 64>);
    else if (dkt == 128) launch(delta_scan_kernel<T, 128>);
    else launch(delta_scan_kernel<T, 256>);
    return check_launch("b200_delta_scan");
  });
}

int b200_head_rmsnorm_gated(void* out, const float* x, const void* weight, const void* gate, int64_t gate_stride, float eps,
                            int64_t n_tok, int H, int dv, int dtype, void* stream) {
  if (n_tok < 0 || H <= 0 || dv <= 0) return fail(B200_EINVAL, "b200_head_rmsnorm_gated: bad sizes");
  if (n_tok == 0) return 0;
  if (!out || !x || !weight) return fail(B200_EINVAL, "b200_head_rmsnorm_gated: null pointer");
  const int64_t rows = n_tok * H;
  return hybrid_by_dtype(dtype, "b200_head_rmsnorm_gated", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    head_rmsnorm_gated_kernel<T><<<static_cast<unsigned>((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(out), x, static_cast<const T*>(weight), static_cast<const T*>(gate), gate_stride, eps, rows, H, dv);
    return check_launch("b200_head_rmsnorm_gated");
  });
}

}  // extern "C"
