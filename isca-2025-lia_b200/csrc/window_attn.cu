// Softmax attention over a sliding window of cached keys and values, with grouped key/value heads, a per-head temperature
// and a tanh soft cap on the scores; no positional rotation (positions enter only through the window).
//
//   kv_store:     the new tokens' keys go into the key cache as they are; each value head is divided by its root mean square
//                 (fp32) and cached so.
//   window_attn:  one block per (token row, group of up to 8 query heads); warp = head.  32 cached positions at a time are
//                 staged in shared memory as fp32 for the key/value heads the block's query heads use; lane j scores key j,
//                     s = cap * tanh((q . k) * scale * temp_h / cap)        (cap <= 0: no cap)
//                 over the positions j with 0 <= pos - j < window, folds the tile into a running softmax and accumulates the
//                 values (lane l owns channels l, l + 32, ...).  Scores, weights and sums are fp32.
#include <math.h>

#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// meta[row] = {slot, position}.  Block per row, warp per value head in turn.
template <typename T>
__global__ void __launch_bounds__(128) kv_store_kernel(const T* __restrict__ k, int ldk, const T* __restrict__ v, int ldv, const int* __restrict__ meta,
                                                       T* __restrict__ kcache, long long k_slot_stride, T* __restrict__ vcache, long long v_slot_stride,
                                                       int G, int dim, int vdim, float eps, int norm_values) {
  const int row = blockIdx.x;
  const int slot = meta[2 * row], pos = meta[2 * row + 1];
  T* kr = kcache + (size_t)slot * k_slot_stride + (size_t)pos * G * dim;
  T* vr = vcache + (size_t)slot * v_slot_stride + (size_t)pos * G * vdim;
  for (int i = threadIdx.x; i < G * dim; i += 128) kr[i] = k[(size_t)row * ldk + i];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = warp; g < G; g += 4) {
    const T* src = v + (size_t)row * ldv + g * vdim;
    float inv = 1.0f;
    if (norm_values) {
      float ss = 0.f;
      for (int c = lane; c < vdim; c += 32) {
        const float x = ldf(src + c);
        ss += x * x;
      }
      inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    }
    for (int c = lane; c < vdim; c += 32) stf(vr + g * vdim + c, ldf(src + c) * inv);
  }
}

constexpr int TK = 32;     // cached positions per stage (= lanes: lane j scores key j)

struct WindowArgs {
  int H, G, dim, vdim, window, HB, NG;       // HB query heads (= warps) per block, spanning at most NG key/value heads
  float scale, softcap;
};

template <typename T, int VR>
__global__ void __launch_bounds__(256) window_attn_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ kcache, long long k_slot_stride,
                                                          const T* __restrict__ vcache, long long v_slot_stride, const int* __restrict__ meta,
                                                          const float* __restrict__ temp, T* __restrict__ out, WindowArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int DKS = a.dim | 1;                     // odd row stride: lanes (= keys) read one channel without bank conflicts
  float* qs = sm;                                // [HB][dim]
  float* ks = qs + a.HB * a.dim;                 // [NG][TK][DKS]
  float* vs = ks + a.NG * TK * DKS;              // [NG][TK][vdim]
  float* ps = vs + a.NG * TK * a.vdim;           // [HB][TK]
  const int row = blockIdx.x, h0 = blockIdx.y * a.HB;
  const int nh = min(a.HB, a.H - h0), rep = a.H / a.G;
  const int g_lo = h0 / rep, ng = (h0 + nh - 1) / rep - g_lo + 1;
  const int slot = meta[2 * row], pos = meta[2 * row + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nthreads = a.HB * 32;
  const int h = h0 + warp;
  const bool live = warp < nh;
  const int gi = live ? h / rep - g_lo : 0;
  const T* kc = kcache + (size_t)slot * k_slot_stride;
  const T* vc = vcache + (size_t)slot * v_slot_stride;

  for (int e = threadIdx.x; e < nh * a.dim; e += nthreads) qs[e] = ldf(q + (size_t)row * ldq + (size_t)h0 * a.dim + e);
  const float sc_mul = live ? a.scale * temp[h] : 0.f;
  float acc[VR];
#pragma unroll
  for (int i = 0; i < VR; ++i) acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  const int j_begin = max(0, pos - a.window + 1);
  for (int j0 = j_begin; j0 <= pos; j0 += TK) {
    __syncthreads();                             // previous stage fully consumed (and qs written, first time)
    const int nk = min(TK, pos + 1 - j0);
    for (int e = threadIdx.x; e < ng * TK * a.dim; e += nthreads) {
      const int g = e / (TK * a.dim), r = e - g * TK * a.dim;
      const int j = r / a.dim, d = r - j * a.dim;
      ks[(g * TK + j) * DKS + d] = j < nk ? ldf(kc + (size_t)(j0 + j) * a.G * a.dim + (g_lo + g) * a.dim + d) : 0.f;
    }
    for (int e = threadIdx.x; e < ng * TK * a.vdim; e += nthreads) {
      const int g = e / (TK * a.vdim), r = e - g * TK * a.vdim;
      const int j = r / a.vdim, c = r - j * a.vdim;
      vs[(g * TK + j) * a.vdim + c] = j < nk ? ldf(vc + (size_t)(j0 + j) * a.G * a.vdim + (g_lo + g) * a.vdim + c) : 0.f;
    }
    __syncthreads();
    if (live) {
      const float* kr = ks + (gi * TK + lane) * DKS;
      const float* qr = qs + warp * a.dim;
      float dot = 0.f;
      for (int d = 0; d < a.dim; ++d) dot = fmaf(qr[d], kr[d], dot);
      float sc = dot * sc_mul;
      if (a.softcap > 0.f) sc = a.softcap * tanhf(sc / a.softcap);
      if (lane >= nk) sc = -INFINITY;
      const float m_new = fmaxf(m_run, warp_max(sc));          // finite: the stage holds at least one visible key
      const float pr = expf(sc - m_new);
      const float al = expf(m_run - m_new);
      l_run = l_run * al + warp_sum(pr);
      m_run = m_new;
      ps[warp * TK + lane] = pr;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < VR; ++i) acc[i] *= al;
      const float* vr = vs + gi * TK * a.vdim;
      for (int j = 0; j < nk; ++j) {
        const float pw = ps[warp * TK + j];
#pragma unroll
        for (int i = 0; i < VR; ++i) {
          const int c = lane + 32 * i;
          if (c < a.vdim) acc[i] = fmaf(pw, vr[j * a.vdim + c], acc[i]);
        }
      }
      __syncwarp();
    }
  }
  if (live) {
    const float invl = 1.0f / l_run;
#pragma unroll
    for (int i = 0; i < VR; ++i) {
      const int c = lane + 32 * i;
      if (c < a.vdim) stf(out + (size_t)row * a.H * a.vdim + (size_t)h * a.vdim + c, acc[i] * invl);
    }
  }
}

size_t attn_smem(const WindowArgs& a) {
  return ((size_t)a.HB * a.dim + (size_t)a.NG * TK * ((a.dim | 1) + a.vdim) + (size_t)a.HB * TK) * sizeof(float);
}

template <typename T, int VR>
int launch_attn(const void* q, int ldq, const void* kcache, long long kss, const void* vcache, long long vss, const int* meta, const float* temp,
                void* out, int M, const WindowArgs& a, cudaStream_t stream) {
  const size_t smem = attn_smem(a);
  if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(window_attn_kernel<T, VR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(M, (a.H + a.HB - 1) / a.HB);
  window_attn_kernel<T, VR><<<grid, a.HB * 32, smem, stream>>>(reinterpret_cast<const T*>(q), ldq, reinterpret_cast<const T*>(kcache), kss,
                                                              reinterpret_cast<const T*>(vcache), vss, meta, temp, reinterpret_cast<T*>(out), a);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

template <typename T>
int dispatch_attn(const void* q, int ldq, const void* kcache, long long kss, const void* vcache, long long vss, const int* meta, const float* temp,
                  void* out, int M, const WindowArgs& a, cudaStream_t stream) {
  if (a.vdim <= 32) return launch_attn<T, 1>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, M, a, stream);
  if (a.vdim <= 64) return launch_attn<T, 2>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, M, a, stream);
  if (a.vdim <= 128) return launch_attn<T, 4>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, M, a, stream);
  if (a.vdim <= 256) return launch_attn<T, 8>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, M, a, stream);
  return launch_attn<T, 16>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, M, a, stream);
}

}  // namespace

extern "C" int lia_kv_store(const void* k, int ldk, const void* v, int ldv, int act_f32, const int* meta, void* kcache, long long k_slot_stride,
                            void* vcache, long long v_slot_stride, int M, int G, int dim, int vdim, float eps, int norm_values,
                            lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(k && v && meta && kcache && vcache && M > 0 && G > 0 && dim > 0 && vdim > 0 && ldk >= G * dim && ldv >= G * vdim, "lia_kv_store: bad arguments");
  if (act_f32)
    kv_store_kernel<float><<<M, 128, 0, stream>>>(reinterpret_cast<const float*>(k), ldk, reinterpret_cast<const float*>(v), ldv, meta,
                                                  reinterpret_cast<float*>(kcache), k_slot_stride, reinterpret_cast<float*>(vcache), v_slot_stride, G, dim, vdim, eps, norm_values);
  else
    kv_store_kernel<bf16><<<M, 128, 0, stream>>>(reinterpret_cast<const bf16*>(k), ldk, reinterpret_cast<const bf16*>(v), ldv, meta,
                                                 reinterpret_cast<bf16*>(kcache), k_slot_stride, reinterpret_cast<bf16*>(vcache), v_slot_stride, G, dim, vdim, eps, norm_values);
  LIA_LAUNCH_CHECK();
  return LIA_OK;
}

extern "C" int lia_window_attn(const void* q, int ldq, int act_f32, const void* kcache, long long k_slot_stride, const void* vcache,
                               long long v_slot_stride, const int* meta, const float* temp, void* out, int M, int H, int G, int dim, int vdim,
                               int window, float scale, float softcap, lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(q && kcache && vcache && meta && temp && out, "lia_window_attn: null pointer");
  LIA_CHECK_ARG(M > 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && vdim <= 512 && window > 0 && H <= 65535 && ldq >= H * dim,
                "lia_window_attn: bad shape H=%d G=%d dim=%d vdim=%d window=%d", H, G, dim, vdim, window);
  WindowArgs a{H, G, dim, vdim, window, 0, 0, scale, softcap};
  // query heads per block: whole groups of `rep` heads while they fit 8 warps, else a divisor of rep (one key/value head)
  const int rep = H / G;
  if (rep >= 8) {
    a.HB = 8;
    while (rep % a.HB) --a.HB;
    a.NG = 1;
  } else {
    a.NG = 8 / rep < G ? 8 / rep : G;
    a.HB = a.NG * rep;
  }
  while (a.NG > 1 && attn_smem(a) > 96 * 1024) {
    --a.NG;
    a.HB = a.NG * rep;
  }
  LIA_CHECK_ARG(attn_smem(a) <= 200 * 1024, "lia_window_attn: heads of %d + %d numbers do not fit the shared-memory stage", dim, vdim);
  if (act_f32) return dispatch_attn<float>(q, ldq, kcache, k_slot_stride, vcache, v_slot_stride, meta, temp, out, M, a, stream);
  return dispatch_attn<bf16>(q, ldq, kcache, k_slot_stride, vcache, v_slot_stride, meta, temp, out, M, a, stream);
}
