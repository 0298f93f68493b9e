// Attention over a compressed (latent) key/value cache.  A token caches ONE row per layer: its normalised latent c
// (kv_rank numbers) followed by one rotated key part (rot numbers) shared by all heads.  Keys and values of a head are
// linear in c (k_h = Wuk_h c, v_h = Wuv_h c), so the kernels never expand them: the query of head h is carried into the
// latent space once (q~_h = Wuk_h^T q_h, a small batched projection made by the caller) and
//     score(t, s, h) = (q~_{t,h} . c_s + qrot_{t,h} . krot_s) * scale,     out~_{t,h} = sum_s softmax_s(score) c_s,
// after which the caller applies Wuv_h to out~.  Per cached token the kernel reads kv_rank + rot numbers whatever the
// number of heads.  Scores, softmax weights and the weighted sums are fp32.
//
//   latent_prep:  RMS-norm of the latent part with its per-channel weight, rotary embedding ("rotate half": channel i is
//                 paired with i + dims/2) of the shared key part at the token's position, both written into the cache row;
//                 the same rotation of each head's rotated query part, written behind that head's q~ slot.
//   latent_attn:  one block per (token, group of up to 8 heads); 32 cached rows at a time are staged in shared memory as
//                 fp32, scored by all heads of the group, folded into a running softmax, and accumulated.
#include <math.h>

#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// rotate-half rotary embedding of `src[0..n)` at position `pos`: the first `dims` channels are rotated, the rest copied.
// inv_freq[i] = base^(-2i/dims), i < dims/2 (fp32, made on the host); the angle pos * inv_freq[i] is an fp32 product.
__device__ __forceinline__ float rotate_half(const float* src, int j, int dims, float pos, const float* inv_freq) {
  if (j >= dims) return src[j];
  const int half = dims >> 1;
  const int i = j < half ? j : j - half;
  const float ang = pos * inv_freq[i];
  const float c = cosf(ang), s = sinf(ang);
  return j < half ? src[j] * c - src[j + half] * s : src[j] * c + src[j - half] * s;
}

// meta[row] = {slot, position}.  Block per token row.
template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(const T* __restrict__ qin, int ldq, const T* __restrict__ dkv, int ldd,
                                                          const float* __restrict__ cw, const float* __restrict__ inv_freq, const int* __restrict__ meta,
                                                          T* __restrict__ cache, long long slot_stride, float* __restrict__ qa, int H, int dim, int rot,
                                                          int rot_dims, int kv_rank, float eps) {
  extern __shared__ float sh[];                 // rot floats: one vector to rotate
  __shared__ float red[4];
  const int row = blockIdx.x;
  const int slot = meta[2 * row], p = meta[2 * row + 1];
  const float pos = (float)p;
  const int D = kv_rank + rot;
  const T* d = dkv + (size_t)row * ldd;
  T* crow = cache + (size_t)slot * slot_stride + (size_t)p * D;

  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += 128) {
    const float v = ldf(d + i);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  for (int i = threadIdx.x; i < rot; i += 128) sh[i] = ldf(d + kv_rank + i);
  __syncthreads();
  const float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < kv_rank; i += 128) stf(crow + i, ldf(d + i) * inv * cw[i]);
  for (int i = threadIdx.x; i < rot; i += 128) stf(crow + kv_rank + i, rotate_half(sh, i, rot_dims, pos, inv_freq));
  for (int h = 0; h < H; ++h) {
    __syncthreads();
    for (int i = threadIdx.x; i < rot; i += 128) sh[i] = ldf(qin + (size_t)row * ldq + h * (dim + rot) + dim + i);
    __syncthreads();
    for (int i = threadIdx.x; i < rot; i += 128) qa[((size_t)row * H + h) * D + kv_rank + i] = rotate_half(sh, i, rot_dims, pos, inv_freq);
  }
}

constexpr int TK = 32;     // cached rows per stage (= one warp's lanes in the softmax step)
constexpr int HG = 8;      // heads per block (= warps per block)

// qa [M][H][D] fp32, cache [slot][capacity][D], out [M][H][kv_rank] fp32, times gate[M][H] (a per-head output gate) if given.  RM = ceil(kv_rank / 256).
template <typename T, int RM>
__global__ void __launch_bounds__(256) latent_attn_kernel(const float* __restrict__ qa, const T* __restrict__ cache, long long slot_stride,
                                                          const int* __restrict__ meta, const float* __restrict__ gate, float* __restrict__ out, int H,
                                                          int kv_rank, int rot, float scale) {
  extern __shared__ float sm[];
  const int D = kv_rank + rot;
  float* qs = sm;                    // [HG][D]
  float* ks = qs + HG * D;           // [TK][D]
  float* ps = ks + TK * D;           // [HG][TK]
  float* alpha = ps + HG * TK;       // [HG]
  float* lsum = alpha + HG;          // [HG]
  const int row = blockIdx.x, h0 = blockIdx.y * HG;
  const int nh = min(HG, H - h0);
  const int slot = meta[2 * row], pos = meta[2 * row + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* crows = cache + (size_t)slot * slot_stride;

  for (int e = threadIdx.x; e < HG * D; e += 256) {
    const int hh = e / D;
    qs[e] = hh < nh ? qa[((size_t)row * H + h0) * D + e] : 0.f;
  }
  float acc[HG][RM];
#pragma unroll
  for (int hh = 0; hh < HG; ++hh)
#pragma unroll
    for (int i = 0; i < RM; ++i) acc[hh][i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;          // of head `warp`, identical in all its lanes

  for (int j0 = 0; j0 <= pos; j0 += TK) {
    __syncthreads();                             // previous stage fully consumed (and qs written, first time)
    const int nk = min(TK, pos + 1 - j0);
    for (int e = threadIdx.x; e < TK * D; e += 256) {
      const int j = e / D;
      ks[e] = j < nk ? ldf(crows + (size_t)j0 * D + e) : 0.f;
    }
    __syncthreads();
    for (int p = warp; p < nh * TK; p += 8) {
      const int hh = p / TK, j = p - hh * TK;
      float dot = 0.f;
      for (int d = lane; d < D; d += 32) dot = fmaf(qs[hh * D + d], ks[j * D + d], dot);
      dot = warp_sum(dot);
      if (lane == 0) ps[p] = j < nk ? dot * scale : -INFINITY;
    }
    __syncthreads();
    if (warp < nh) {
      const float s = ps[warp * TK + lane];
      const float m_new = fmaxf(m_run, warp_max(s));          // finite: the stage holds at least one visible key
      const float pr = expf(s - m_new);
      const float a = expf(m_run - m_new);
      l_run = l_run * a + warp_sum(pr);
      m_run = m_new;
      ps[warp * TK + lane] = pr;
      if (lane == 0) alpha[warp] = a;
    }
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) {
      const float a = hh < nh ? alpha[hh] : 0.f;
#pragma unroll
      for (int i = 0; i < RM; ++i) acc[hh][i] *= a;
    }
    for (int j = 0; j < nk; ++j) {
      float kv[RM];
#pragma unroll
      for (int i = 0; i < RM; ++i) {
        const int r = threadIdx.x + 256 * i;
        kv[i] = r < kv_rank ? ks[j * D + r] : 0.f;
      }
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) {
        const float pw = ps[hh * TK + j];                       // rows of absent heads hold stale values: never stored
#pragma unroll
        for (int i = 0; i < RM; ++i) acc[hh][i] = fmaf(pw, kv[i], acc[hh][i]);
      }
    }
  }
  if (warp < nh && lane == 0) lsum[warp] = l_run;
  __syncthreads();
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) {
    if (hh < nh) {
      const float invl = (gate ? gate[(size_t)row * H + h0 + hh] : 1.0f) / lsum[hh];
#pragma unroll
      for (int i = 0; i < RM; ++i) {
        const int r = threadIdx.x + 256 * i;
        if (r < kv_rank) out[((size_t)row * H + h0 + hh) * kv_rank + r] = acc[hh][i] * invl;
      }
    }
  }
}

template <typename T, int RM>
int launch_attn(const float* qa, const void* cache, long long slot_stride, const int* meta, const float* gate, float* out, int M, int H, int kv_rank, int rot,
                float scale, cudaStream_t stream) {
  const int D = kv_rank + rot;
  const size_t smem = ((size_t)HG * D + (size_t)TK * D + HG * TK + 2 * HG) * sizeof(float);
  LIA_CHECK_ARG(smem <= 200 * 1024, "lia_latent_attn: a cache row of %d numbers does not fit the shared-memory stage", D);
  if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(latent_attn_kernel<T, RM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(M, (H + HG - 1) / HG);
  latent_attn_kernel<T, RM><<<grid, 256, smem, stream>>>(qa, reinterpret_cast<const T*>(cache), slot_stride, meta, gate, out, H, kv_rank, rot, scale);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

template <typename T>
int dispatch_attn(const float* qa, const void* cache, long long slot_stride, const int* meta, const float* gate, float* out, int M, int H, int kv_rank, int rot,
                  float scale, cudaStream_t stream) {
  if (kv_rank <= 256) return launch_attn<T, 1>(qa, cache, slot_stride, meta, gate, out, M, H, kv_rank, rot, scale, stream);
  if (kv_rank <= 512) return launch_attn<T, 2>(qa, cache, slot_stride, meta, gate, out, M, H, kv_rank, rot, scale, stream);
  return launch_attn<T, 4>(qa, cache, slot_stride, meta, gate, out, M, H, kv_rank, rot, scale, stream);
}

}  // namespace

extern "C" int lia_latent_prep(const void* q, int ldq, const void* dkv, int ldd, int act_f32, const float* c_norm_w, const float* inv_freq,
                               const int* meta, void* cache, long long slot_stride, float* qa, int M, int H, int dim, int rot, int rot_dims,
                               int kv_rank, float eps, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(q && dkv && c_norm_w && inv_freq && meta && cache && qa, "lia_latent_prep: null pointer");
  LIA_CHECK_ARG(M > 0 && H > 0 && dim >= 0 && rot > 0 && kv_rank > 0 && rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0 && rot <= 8192,
                "lia_latent_prep: bad shape H=%d dim=%d rot=%d rot_dims=%d kv_rank=%d", H, dim, rot, rot_dims, kv_rank);
  const size_t smem = (size_t)rot * sizeof(float);
  if (act_f32)
    latent_prep_kernel<float><<<M, 128, smem, stream>>>(reinterpret_cast<const float*>(q), ldq, reinterpret_cast<const float*>(dkv), ldd, c_norm_w, inv_freq,
                                                        meta, reinterpret_cast<float*>(cache), slot_stride, qa, H, dim, rot, rot_dims, kv_rank, eps);
  else
    latent_prep_kernel<bf16><<<M, 128, smem, stream>>>(reinterpret_cast<const bf16*>(q), ldq, reinterpret_cast<const bf16*>(dkv), ldd, c_norm_w, inv_freq,
                                                       meta, reinterpret_cast<bf16*>(cache), slot_stride, qa, H, dim, rot, rot_dims, kv_rank, eps);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_latent_attn(const float* qa, const void* cache, int cache_f32, long long slot_stride, const int* meta, const float* gate,
                               float* out, int M, int H, int kv_rank, int rot, float scale, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(qa && cache && meta && out, "lia_latent_attn: null pointer");
  LIA_CHECK_ARG(M > 0 && H > 0 && H <= 65535 * HG && kv_rank > 0 && kv_rank <= 1024 && rot >= 0, "lia_latent_attn: bad shape M=%d H=%d kv_rank=%d rot=%d", M, H, kv_rank, rot);
  if (cache_f32) return dispatch_attn<float>(qa, cache, slot_stride, meta, gate, out, M, H, kv_rank, rot, scale, stream);
  return dispatch_attn<bf16>(qa, cache, slot_stride, meta, gate, out, M, H, kv_rank, rot, scale, stream);
}
