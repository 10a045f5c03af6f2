// Pieces for decoder designs whose sublayers read the fp32 residual stream itself, are gated by a sigmoid of a linear
// map of that stream and are normed on the way out:
//
//   token shift                  h_t <- h_t + (h_(t-1) - h_t) * mu per channel, with the unshifted previous row; the last
//                                row of every live sequence is carried in a slot pool
//   latent rotary append         a latent attention with a decoupled rotated key part: the first `rank` columns of the
//                                down-projection are RMS-normed, the last `dr` are turned by the position (shared by all
//                                heads), both go to one row of a one-head pool; the rotated part of every query head is
//                                turned the same way.  Frequencies come from the caller (any rescaling is the caller's);
//                                cos and sin carry a common gain
//   head difference norm         o = a1 - lambda a2 of two score maps over the same values, unit RMS per head, times a
//                                constant
//   gated post-norm residual     x += (offset + w) * N(a * sigmoid(g)) on the fp32 residual
//   squared ReLU                 y = max(z, 0)^2
//   gated table rows             g = gelu_tanh(z) * table[token][col0 ...]: a per-layer slice of a second embedding table
//                                gated by a projection of the residual
//   router logits                fp32 x . W^T + b for few outputs, summed in an order that depends on the width alone
//
// Every size and constant of a design is a parameter.  Norm statistics, angles, gates and the residual are fp32 whatever
// the storage dtype T is.
#include <algorithm>
#include <type_traits>

#include "../../include/b200_mixers.h"
#include "b200_common.cuh"

namespace b200 {
namespace {

template <typename F>
int gated_by_dtype(int dtype, const char* name, F&& f) {
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

__device__ __forceinline__ float block_sum_all(float v, float* red) {
  // every thread returns the total; `red` holds 32 floats
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

struct SeqSpan {
  int tok0;   // first packed row
  int count;  // tokens in this step
  int slot;   // state slot
  int fresh;  // 1: the sequence starts here (the carried row counts as zero)
};

// ---- token shift ---------------------------------------------------------------------------------------------------
// Grid (sequence, run of kShiftTokens tokens, 128 channels); a thread walks its run for one channel with the previous
// row's value in a register.  The thread that serves a sequence's FIRST run reads the carried row and afterwards stores
// the sequence's last row of this step in its place, so the slot is read and written by the same thread, in that order.
constexpr int kShiftTokens = 32;

template <typename T>
__global__ void __launch_bounds__(128)
token_shift_kernel(T* __restrict__ out, int64_t out_stride, T* __restrict__ x_cast, const float* __restrict__ x,
                   const T* __restrict__ mu, float* __restrict__ state, const SeqSpan* __restrict__ seqs, int W) {
  const SeqSpan sq = seqs[blockIdx.x];
  const int t0 = blockIdx.y * kShiftTokens;
  if (t0 >= sq.count) return;
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  if (c >= W) return;
  const float m = Cvt<T>::to_f32(mu[c]);
  const float* xr = x + static_cast<int64_t>(sq.tok0) * W + c;
  float prev;
  if (t0 > 0) prev = xr[static_cast<int64_t>(t0 - 1) * W];
  else prev = sq.fresh ? 0.f : state[static_cast<int64_t>(sq.slot) * W + c];
  const int t1 = min(sq.count, t0 + kShiftTokens);
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    const float cur = xr[static_cast<int64_t>(t) * W];
    out[static_cast<int64_t>(sq.tok0 + t) * out_stride + c] = Cvt<T>::from_f32(fmaf(prev - cur, m, cur));
    if (x_cast) x_cast[static_cast<int64_t>(sq.tok0 + t) * W + c] = Cvt<T>::from_f32(cur);
    prev = cur;
  }
  if (t0 == 0) state[static_cast<int64_t>(sq.slot) * W + c] = xr[static_cast<int64_t>(sq.count - 1) * W];
}

// ---- latent rotary append ------------------------------------------------------------------------------------------
// One CTA per token.  (cos, sin) * gain of the token's angles are formed once (double precision angles) and serve the
// shared key part and every query head.
template <typename T>
__global__ void __launch_bounds__(128)
latent_rotary_append_kernel(const T* __restrict__ q_rot, int64_t q_tok_stride, int64_t q_head_stride, T* __restrict__ q_out,
                            int64_t qo_tok_stride, int64_t qo_head_stride, const T* __restrict__ dkv, int64_t dkv_stride,
                            const T* __restrict__ w_c, float eps, const double* __restrict__ freqs, float gain, int rot_dims,
                            T* __restrict__ pool, const int64_t* __restrict__ slot_mapping,
                            const int32_t* __restrict__ tok_pos, int H, int dr, int rank) {
  extern __shared__ float cs[];   // [rot_dims / 2][2]
  __shared__ float red[32];
  const int64_t n = blockIdx.x;
  const int half = rot_dims / 2;
  const int p = tok_pos[n];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double s, c;
    sincos(static_cast<double>(p) * freqs[i], &s, &c);
    cs[2 * i] = static_cast<float>(c) * gain;
    cs[2 * i + 1] = static_cast<float>(s) * gain;
  }
  const T* row = dkv + n * dkv_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = Cvt<T>::to_f32(row[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = rsqrtf(block_sum_all(ss, red) / static_cast<float>(rank) + eps);   // its barriers also publish cs
  const int64_t slot = slot_mapping[n];
  if (slot >= 0) {
    T* dst = pool + slot * (rank + dr);
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
      dst[i] = Cvt<T>::from_f32(Cvt<T>::to_f32(row[i]) * inv * Cvt<T>::to_f32(w_c[i]));
    for (int i = threadIdx.x; i < dr; i += blockDim.x) {
      float y = Cvt<T>::to_f32(row[rank + i]);
      if (i < rot_dims) {
        const float other = Cvt<T>::to_f32(row[rank + (i ^ 1)]);
        const float c = cs[i & ~1], s = cs[i | 1];
        y = (i & 1) ? fmaf(y, c, other * s) : fmaf(y, c, -other * s);   // (u, v) -> (u c - v s, v c + u s)
      }
      dst[rank + i] = Cvt<T>::from_f32(y);
    }
  }
  const T* qs = q_rot + n * q_tok_stride;
  T* qd = q_out + n * qo_tok_stride;
  for (int e = threadIdx.x; e < H * dr; e += blockDim.x) {
    const int h = e / dr, i = e - h * dr;
    float y = Cvt<T>::to_f32(qs[h * q_head_stride + i]);
    if (i < rot_dims) {
      const float other = Cvt<T>::to_f32(qs[h * q_head_stride + (i ^ 1)]);
      const float c = cs[i & ~1], s = cs[i | 1];
      y = (i & 1) ? fmaf(y, c, other * s) : fmaf(y, c, -other * s);
    }
    qd[h * qo_head_stride + i] = Cvt<T>::from_f32(y);
  }
}

// ---- head difference norm ------------------------------------------------------------------------------------------
// One warp per (token, head).  The two maps of head h sit at heads (h / rep) * 2 rep + (h % rep) and that + rep of `a`.
template <typename T, typename A>
__global__ void __launch_bounds__(256)
head_diff_norm_kernel(T* __restrict__ out, int64_t out_stride, const A* __restrict__ a, int64_t a_tok_stride,
                      int64_t a_head_stride, float lam, float out_scale, float eps, int64_t rows, int H, int rep, int dv) {
  const int64_t r = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t n = r / H;
  const int h = static_cast<int>(r - n * H);
  const A* a1 = a + n * a_tok_stride + ((h / rep) * 2 * rep + (h % rep)) * a_head_stride;
  const A* a2 = a1 + rep * a_head_stride;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) {
    const float o = fmaf(-lam, Cvt<A>::to_f32(a2[i]), Cvt<A>::to_f32(a1[i]));
    ss = fmaf(o, o, ss);
  }
  const float f = rsqrtf(warp_sum(ss) / static_cast<float>(dv) + eps) * out_scale;
  T* dst = out + n * out_stride + static_cast<int64_t>(h) * dv;
  for (int i = lane; i < dv; i += 32)
    dst[i] = Cvt<T>::from_f32(fmaf(-lam, Cvt<A>::to_f32(a2[i]), Cvt<A>::to_f32(a1[i])) * f);
}

// ---- gated post-norm residual --------------------------------------------------------------------------------------
template <typename T, typename A>
__global__ void __launch_bounds__(256)
gated_postnorm_residual_kernel(float* __restrict__ x, const A* __restrict__ a, int64_t a_stride, const T* __restrict__ g,
                               int64_t g_stride, const T* __restrict__ w, float w_off, T* __restrict__ x_out, float eps,
                               int width) {
  extern __shared__ float gp_row[];
  __shared__ float red[32];
  const int64_t n = blockIdx.x;
  const A* ar = a + n * a_stride;
  const T* gr = g ? g + n * g_stride : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float y = Cvt<A>::to_f32(ar[i]);
    if (gr) y *= sigmoidf_(Cvt<T>::to_f32(gr[i]));
    gp_row[i] = y;
    ss = fmaf(y, y, ss);
  }
  const float inv = rsqrtf(block_sum_all(ss, red) / static_cast<float>(width) + eps);
  float* xr = x + n * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float s = xr[i] + gp_row[i] * inv * (w_off + Cvt<T>::to_f32(w[i]));
    xr[i] = s;
    if (x_out) x_out[n * width + i] = Cvt<T>::from_f32(s);
  }
}

// ---- squared ReLU --------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
relu_squared_kernel(T* __restrict__ out, const T* __restrict__ z, int64_t z_stride, int64_t rows, int ff) {
  const int64_t total = rows * ff;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = e / ff;
    const int c = static_cast<int>(e - r * ff);
    const float v = fmaxf(Cvt<T>::to_f32(z[r * z_stride + c]), 0.f);
    out[e] = Cvt<T>::from_f32(v * v);
  }
}

// 16-byte accesses when the rows allow
template <typename T>
__global__ void __launch_bounds__(256)
relu_squared_vec_kernel(T* __restrict__ out, const T* __restrict__ z, int64_t z_stride, int64_t rows, int ff) {
  constexpr int E = 16 / sizeof(T);
  const int per_row = ff / E;
  const int64_t total = rows * per_row;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = e / per_row;
    const int c = static_cast<int>(e - r * per_row) * E;
    int4 raw = *reinterpret_cast<const int4*>(z + r * z_stride + c);
    T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int u = 0; u < E; ++u) {
      const float f = fmaxf(Cvt<T>::to_f32(v[u]), 0.f);
      v[u] = Cvt<T>::from_f32(f * f);
    }
    *reinterpret_cast<int4*>(out + r * ff + c) = raw;
  }
}

// ---- gated table rows ----------------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_tanh_(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_table_rows_kernel(T* __restrict__ out, const T* __restrict__ z, int64_t z_stride, const T* __restrict__ table,
                        int64_t table_stride, int col0, const int64_t* __restrict__ tokens, int64_t n_tok, int d) {
  const int64_t total = n_tok * d;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t n = e / d;
    const int c = static_cast<int>(e - n * d);
    const float row = Cvt<T>::to_f32(table[tokens[n] * table_stride + col0 + c]);
    out[e] = Cvt<T>::from_f32(gelu_tanh_(Cvt<T>::to_f32(z[n * z_stride + c])) * row);
  }
}

// ---- router logits -------------------------------------------------------------------------------------------------
// One CTA of four warps per token, kRouterChunk experts at a time: thread t owns columns t, t + 128, ... (four at a time
// when the width allows); partial sums meet in a butterfly per warp and the four warps' sums are added in warp order.
// The order of every sum depends on the width alone, so a token's logits - and with them its experts - do not depend on
// what else the step carries.
constexpr int kRouterChunk = 8;
constexpr int kRouterThreads = 128;

template <bool VEC>
__global__ void __launch_bounds__(kRouterThreads)
router_logits_kernel(float* __restrict__ logits, const float* __restrict__ x, const float* __restrict__ w,
                     const float* __restrict__ bias, int E, int W) {
  __shared__ float part[kRouterThreads / 32][kRouterChunk];
  const int64_t n = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* xr = x + n * W;
  for (int e0 = 0; e0 < E; e0 += kRouterChunk) {
    float acc[kRouterChunk];
#pragma unroll
    for (int j = 0; j < kRouterChunk; ++j) acc[j] = 0.f;
    if (VEC) {
      for (int i = threadIdx.x * 4; i < W; i += kRouterThreads * 4) {
        const float4 xv = *reinterpret_cast<const float4*>(xr + i);
#pragma unroll
        for (int j = 0; j < kRouterChunk; ++j)
          if (e0 + j < E) {
            const float4 wv = *reinterpret_cast<const float4*>(w + static_cast<int64_t>(e0 + j) * W + i);
            acc[j] = fmaf(xv.x, wv.x, fmaf(xv.y, wv.y, fmaf(xv.z, wv.z, fmaf(xv.w, wv.w, acc[j]))));
          }
      }
    } else {
      for (int i = threadIdx.x; i < W; i += kRouterThreads) {
        const float xv = xr[i];
#pragma unroll
        for (int j = 0; j < kRouterChunk; ++j)
          if (e0 + j < E) acc[j] = fmaf(xv, w[static_cast<int64_t>(e0 + j) * W + i], acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < kRouterChunk; ++j) {
      const float t = warp_sum(acc[j]);
      if (lane == 0) part[warp][j] = t;
    }
    __syncthreads();
    if (threadIdx.x < kRouterChunk && e0 + threadIdx.x < E) {
      float t = part[0][threadIdx.x];
#pragma unroll
      for (int ww = 1; ww < kRouterThreads / 32; ++ww) t += part[ww][threadIdx.x];
      logits[n * E + e0 + threadIdx.x] = t + (bias ? bias[e0 + threadIdx.x] : 0.f);
    }
    __syncthreads();
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_token_shift(void* out, int64_t out_stride, void* x_cast, const float* x, const void* mu, float* state,
                     const int32_t* seqs, int n_seqs, int max_count, int width, int dtype, void* stream) {
  if (n_seqs < 0 || max_count < 0 || width <= 0 || out_stride < width) return fail(B200_EINVAL, "b200_token_shift: bad sizes");
  if (n_seqs == 0 || max_count == 0) return 0;
  if (!out || !x || !mu || !state || !seqs) return fail(B200_EINVAL, "b200_token_shift: null pointer");
  const dim3 grid(n_seqs, (max_count + kShiftTokens - 1) / kShiftTokens, (width + 127) / 128);
  return gated_by_dtype(dtype, "b200_token_shift", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    token_shift_kernel<T><<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(out), out_stride, static_cast<T*>(x_cast), x, static_cast<const T*>(mu), state,
        reinterpret_cast<const SeqSpan*>(seqs), width);
    return check_launch("b200_token_shift");
  });
}

int b200_latent_rotary_append(const void* q_rot, int64_t q_tok_stride, int64_t q_head_stride, void* q_out,
                              int64_t qo_tok_stride, int64_t qo_head_stride, const void* dkv, int64_t dkv_stride,
                              const void* c_norm, float eps, const double* freqs, float gain, int rot_dims, void* pool,
                              const int64_t* slot_mapping, const int32_t* tok_pos, int n_tok, int H, int rot_width,
                              int rank, int dtype, void* stream) {
  if (n_tok < 0 || H <= 0 || rot_width < 0 || rank <= 0 || rot_dims < 0 || rot_dims > rot_width || (rot_dims & 1))
    return fail(B200_EINVAL, "b200_latent_rotary_append: bad sizes");
  if (n_tok == 0) return 0;
  if (!q_rot || !q_out || !dkv || !c_norm || !pool || !slot_mapping || !tok_pos || (rot_dims > 0 && !freqs))
    return fail(B200_EINVAL, "b200_latent_rotary_append: null pointer");
  const size_t smem = sizeof(float) * std::max(rot_dims, 2);
  return gated_by_dtype(dtype, "b200_latent_rotary_append", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    latent_rotary_append_kernel<T><<<n_tok, 128, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const T*>(q_rot), q_tok_stride, q_head_stride, static_cast<T*>(q_out), qo_tok_stride, qo_head_stride,
        static_cast<const T*>(dkv), dkv_stride, static_cast<const T*>(c_norm), eps, freqs, gain, rot_dims,
        static_cast<T*>(pool), slot_mapping, tok_pos, H, rot_width, rank);
    return check_launch("b200_latent_rotary_append");
  });
}

int b200_head_diff_norm(void* out, int64_t out_stride, const void* a, int64_t a_tok_stride, int64_t a_head_stride,
                        int a_is_f32, float lam, float out_scale, float eps, int64_t n_tok, int H, int rep, int dv, int dtype,
                        void* stream) {
  if (n_tok < 0 || H <= 0 || rep <= 0 || H % rep || dv <= 0) return fail(B200_EINVAL, "b200_head_diff_norm: bad sizes");
  if (n_tok == 0) return 0;
  if (!out || !a) return fail(B200_EINVAL, "b200_head_diff_norm: null pointer");
  const int64_t rows = n_tok * H;
  return gated_by_dtype(dtype, "b200_head_diff_norm", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
    auto s = static_cast<cudaStream_t>(stream);
    if (a_is_f32)
      head_diff_norm_kernel<T, float><<<grid, 256, 0, s>>>(static_cast<T*>(out), out_stride, static_cast<const float*>(a),
                                                           a_tok_stride, a_head_stride, lam, out_scale, eps, rows, H, rep, dv);
    else
      head_diff_norm_kernel<T, T><<<grid, 256, 0, s>>>(static_cast<T*>(out), out_stride, static_cast<const T*>(a),
                                                       a_tok_stride, a_head_stride, lam, out_scale, eps, rows, H, rep, dv);
    return check_launch("b200_head_diff_norm");
  });
}

int b200_gated_postnorm_residual(float* x, const void* a, int64_t a_stride, int a_is_f32, const void* gate,
                                 int64_t gate_stride, const void* w_norm, float weight_offset, void* x_out, float eps,
                                 int rows, int width, int dtype, void* stream) {
  if (rows < 0 || width <= 0) return fail(B200_EINVAL, "b200_gated_postnorm_residual: bad sizes");
  if (rows == 0) return 0;
  if (!x || !a || !w_norm) return fail(B200_EINVAL, "b200_gated_postnorm_residual: null pointer");
  const size_t smem = sizeof(float) * static_cast<size_t>(width);
  if (smem > 200 * 1024) return fail(B200_ESHAPE, "b200_gated_postnorm_residual: width %d is too wide", width);
  return gated_by_dtype(dtype, "b200_gated_postnorm_residual", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto launch = [&](auto kern, auto* ap) {
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      kern<<<rows, 256, smem, static_cast<cudaStream_t>(stream)>>>(x, ap, a_stride, static_cast<const T*>(gate), gate_stride,
                                                                   static_cast<const T*>(w_norm), weight_offset,
                                                                   static_cast<T*>(x_out), eps, width);
    };
    if (a_is_f32) launch(gated_postnorm_residual_kernel<T, float>, static_cast<const float*>(a));
    else launch(gated_postnorm_residual_kernel<T, T>, static_cast<const T*>(a));
    return check_launch("b200_gated_postnorm_residual");
  });
}

int b200_relu_squared(void* out, const void* z, int64_t z_stride, int64_t rows, int ff, int dtype, void* stream) {
  if (rows < 0 || ff <= 0 || z_stride < ff) return fail(B200_EINVAL, "b200_relu_squared: bad sizes");
  if (rows == 0) return 0;
  if (!out || !z) return fail(B200_EINVAL, "b200_relu_squared: null pointer");
  const int esz = dtype_size(dtype);
  if (esz == 0) return fail(B200_EINVAL, "b200_relu_squared: unsupported dtype %d", dtype);
  const int E = 16 / esz;
  const bool vec = ff % E == 0 && z_stride % E == 0 && aligned16(out) && aligned16(z);
  const int64_t items = vec ? rows * (ff / E) : rows * ff;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((items + 255) / 256, kNumSMs * 16));
  return gated_by_dtype(dtype, "b200_relu_squared", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    auto s = static_cast<cudaStream_t>(stream);
    if (vec) relu_squared_vec_kernel<T><<<grid, 256, 0, s>>>(static_cast<T*>(out), static_cast<const T*>(z), z_stride, rows, ff);
    else relu_squared_kernel<T><<<grid, 256, 0, s>>>(static_cast<T*>(out), static_cast<const T*>(z), z_stride, rows, ff);
    return check_launch("b200_relu_squared");
  });
}

int b200_gated_table_rows(void* out, const void* z, int64_t z_stride, const void* table, int64_t table_stride, int col0,
                          const int64_t* tokens, int64_t n_tok, int d, int dtype, void* stream) {
  if (n_tok < 0 || d <= 0 || col0 < 0 || table_stride < col0 + d) return fail(B200_EINVAL, "b200_gated_table_rows: bad sizes");
  if (n_tok == 0) return 0;
  if (!out || !z || !table || !tokens) return fail(B200_EINVAL, "b200_gated_table_rows: null pointer");
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((n_tok * d + 255) / 256, kNumSMs * 16));
  return gated_by_dtype(dtype, "b200_gated_table_rows", [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    gated_table_rows_kernel<T><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<T*>(out), static_cast<const T*>(z), z_stride, static_cast<const T*>(table), table_stride, col0, tokens,
        n_tok, d);
    return check_launch("b200_gated_table_rows");
  });
}

int b200_router_logits(float* logits, const float* x, const float* w, const float* bias, int64_t n_tok, int E, int width,
                       void* stream) {
  if (n_tok < 0 || E <= 0 || width <= 0) return fail(B200_EINVAL, "b200_router_logits: bad sizes");
  if (n_tok == 0) return 0;
  if (!logits || !x || !w) return fail(B200_EINVAL, "b200_router_logits: null pointer");
  const unsigned grid = static_cast<unsigned>(n_tok);
  auto s = static_cast<cudaStream_t>(stream);
  if (width % 4 == 0 && aligned16(x) && aligned16(w))
    router_logits_kernel<true><<<grid, kRouterThreads, 0, s>>>(logits, x, w, bias, E, width);
  else
    router_logits_kernel<false><<<grid, kRouterThreads, 0, s>>>(logits, x, w, bias, E, width);
  return check_launch("b200_router_logits");
}

}  // extern "C"
