// Softmax attention over a sliding window of cached keys and values, with grouped key/value heads, a per-head temperature
// and a tanh soft cap on the scores; no positional rotation (positions enter only through the window).
//
//   kv_store:     the new tokens' keys go into the key cache as they are; each value head is divided by its root mean square
//                 (fp32) and cached so.
//   window_attn:  one block per (group of token rows, group of up to 8 query heads, range of keys); a warp owns (row, head)
//                 pairs.  32 cached positions at a time are staged in shared memory as fp32 for the key/value heads the
//                 block's query heads use, once for all rows of the block that continue one sequence; lane j scores key j,
//                     s = cap * tanh((q . k) * scale * temp_h / cap)        (cap <= 0: no cap)
//                 over the positions j with 0 <= pos - j < window, folds the stage into a running softmax and accumulates the
//                 values (lane l owns channels l, l + 32, ...).  Scores, weights and sums are fp32.  Few rows and a long
//                 window (decoding): the keys are split over several blocks and a second kernel combines.
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
constexpr int NWARP = 8;

struct WindowArgs {
  int H, G, dim, vdim, window;
  int HB, NG, QR, nsplit;      // query heads per block (spanning at most NG key/value heads), rows per block, key ranges per row
  float scale, softcap;
};

__host__ __device__ inline int key_stride(int dim) { return dim % 4 == 0 ? dim + 4 : (dim | 1); }   // conflict-free rows (128-bit or scalar reads)

template <typename T> struct Vec { static constexpr int N = 8; };
template <> struct Vec<float> { static constexpr int N = 4; };
__device__ __forceinline__ void load_vec(const bf16* p, float* f) { unpack8(*reinterpret_cast<const uint4*>(p), f); }
__device__ __forceinline__ void load_vec(const float* p, float* f) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}

// rows [n][G][width] of a cache -> shared memory [ng][TK][stride] as fp32, positions j0 .. j0+nk-1 (zeros behind them)
template <typename T>
__device__ __forceinline__ void stage_rows(const T* __restrict__ cache, int G, int width, int g_lo, int ng, int j0, int nk, float* dst, int stride,
                                           bool vec) {
  constexpr int VEC = Vec<T>::N;
  if (vec) {
    const int per_row = width / VEC, total = ng * TK * per_row;
    for (int e = threadIdx.x; e < total; e += NWARP * 32) {
      const int g = e / (TK * per_row), r = e - g * TK * per_row;
      const int j = r / per_row, c = (r - j * per_row) * VEC;
      float f[VEC];
      if (j < nk) {
        load_vec(cache + ((size_t)(j0 + j) * G + g_lo + g) * width + c, f);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = 0.f;
      }
      float* d = dst + (g * TK + j) * stride + c;
#pragma unroll
      for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4*>(d + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
    }
  } else {
    const int total = ng * TK * width;
    for (int e = threadIdx.x; e < total; e += NWARP * 32) {
      const int g = e / (TK * width), r = e - g * TK * width;
      const int j = r / width, c = r - j * width;
      dst[(g * TK + j) * stride + c] = j < nk ? ldf(cache + ((size_t)(j0 + j) * G + g_lo + g) * width + c) : 0.f;
    }
  }
}

// One block: rows [blockIdx.x * QR, + QR) of the step, query heads [blockIdx.y * HB, + HB), the blockIdx.z-th part of the keys.
// Rows that continue one sequence (same slot, consecutive positions) form a run and share the staged keys and values; a block
// whose rows belong to several sequences takes the runs one after the other.  A (row, head) pair belongs to one warp, which
// keeps its running maximum, sum and value accumulators (lane l: channels l, l + 32, ...) in registers; PP pairs per warp.
// nsplit > 1: unnormalised sums to `part` [M][H][nsplit][vdim] and (max, sum) to `part_ml`; window_combine_kernel finishes.
template <typename T, int VR, int PP>
__global__ void __launch_bounds__(NWARP * 32) window_attn_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ kcache, long long k_slot_stride,
                                                                const T* __restrict__ vcache, long long v_slot_stride, const int* __restrict__ meta,
                                                                const float* __restrict__ temp, T* __restrict__ out, float* __restrict__ part,
                                                                float2* __restrict__ part_ml, int M, WindowArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int DKS = key_stride(a.dim);
  float* qs = sm;                                             // [QR * HB][dim]
  float* ks = qs + (a.QR * a.HB * a.dim + 3) / 4 * 4;         // [NG][TK][DKS]
  float* vs = ks + a.NG * TK * DKS;                           // [NG][TK][vdim]
  const int r_begin = blockIdx.x * a.QR, r_end = min(M, r_begin + a.QR);
  const int h0 = blockIdx.y * a.HB, z = blockIdx.z;
  const int nh = min(a.HB, a.H - h0), rep = a.H / a.G;
  const int g_lo = h0 / rep, ng = (h0 + nh - 1) / rep - g_lo + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int VEC = Vec<T>::N;
  const bool aligned = reinterpret_cast<uintptr_t>(kcache) % 16 == 0 && reinterpret_cast<uintptr_t>(vcache) % 16 == 0 &&
                       k_slot_stride % VEC == 0 && v_slot_stride % VEC == 0;
  const bool vec_k = aligned && a.dim % VEC == 0 && a.dim % 4 == 0, vec_v = aligned && a.vdim % VEC == 0;
  const bool dot4 = a.dim % 4 == 0;
  const bool same_head = NWARP % nh == 0 && PP > 1;           // pair p = warp + 8 s belongs to head p % nh = warp % nh for every s

  int r = r_begin;
  while (r < r_end) {
    const int slot = meta[2 * r], pos_first = meta[2 * r + 1];
    int re = r + 1;
    while (re < r_end && meta[2 * re] == slot && meta[2 * re + 1] == pos_first + (re - r)) ++re;
    const int nrun = re - r, npairs = nrun * nh, pos_last = pos_first + nrun - 1;
    const T* kc = kcache + (size_t)slot * k_slot_stride;
    const T* vc = vcache + (size_t)slot * v_slot_stride;
    __syncthreads();                                          // the previous run's queries and stage are no longer read
    for (int e = threadIdx.x; e < npairs * a.dim; e += NWARP * 32) {
      const int p = e / a.dim, d = e - p * a.dim;
      const int i = p / nh, hh = p - i * nh;
      qs[e] = ldf(q + (size_t)(r + i) * ldq + (size_t)(h0 + hh) * a.dim + d);
    }
    float m_run[PP], l_run[PP], acc[PP][VR];
#pragma unroll
    for (int s = 0; s < PP; ++s) {
      m_run[s] = -INFINITY;
      l_run[s] = 0.f;
#pragma unroll
      for (int i = 0; i < VR; ++i) acc[s][i] = 0.f;
    }
    const int jb = max(0, pos_first - a.window + 1);
    const int ntiles = (pos_last - jb) / TK + 1, per = (ntiles + a.nsplit - 1) / a.nsplit;
    const int t_end = min(ntiles, (z + 1) * per);
    for (int t = z * per; t < t_end; ++t) {
      const int j0 = jb + t * TK, nk = min(TK, pos_last + 1 - j0);
      __syncthreads();                                        // previous stage fully consumed (and qs written, first time)
      stage_rows(kc, a.G, a.dim, g_lo, ng, j0, nk, ks, DKS, vec_k);
      stage_rows(vc, a.G, a.vdim, g_lo, ng, j0, nk, vs, a.vdim, vec_v);
      __syncthreads();
      if (same_head) {
        // All pairs of this warp are rows of ONE query head (nh divides the warp count): a staged key or value row is read
        // from shared memory once and serves the PP rows.
        const int hh = warp % nh, h = h0 + hh, gi = h / rep - g_lo;
        const float sc_mul = a.scale * temp[h];
        bool active[PP];
        int lo_min = 0x7fffffff, pos_max = -1;
#pragma unroll
        for (int s = 0; s < PP; ++s) {
          const int p = warp + NWARP * s;
          const int pos = pos_first + p / nh, lo = max(0, pos - a.window + 1);
          active[s] = p < npairs && j0 <= pos && j0 + nk - 1 >= lo;
          if (active[s]) {
            lo_min = min(lo_min, lo);
            pos_max = max(pos_max, pos);
          }
        }
        if (pos_max >= 0) {
          float dot[PP];
#pragma unroll
          for (int s = 0; s < PP; ++s) dot[s] = 0.f;
          const float* kr = ks + (gi * TK + lane) * DKS;
          if (dot4) {
            const float4* k4 = reinterpret_cast<const float4*>(kr);
            for (int d = 0; d < a.dim / 4; ++d) {
              const float4 y = k4[d];
#pragma unroll
              for (int s = 0; s < PP; ++s) {
                const float4 x = reinterpret_cast<const float4*>(qs + (warp + NWARP * s) * a.dim)[d];
                dot[s] = fmaf(x.x, y.x, fmaf(x.y, y.y, fmaf(x.z, y.z, fmaf(x.w, y.w, dot[s]))));
              }
            }
          } else {
            for (int d = 0; d < a.dim; ++d) {
              const float y = kr[d];
#pragma unroll
              for (int s = 0; s < PP; ++s) dot[s] = fmaf(qs[(warp + NWARP * s) * a.dim + d], y, dot[s]);
            }
          }
          float pr[PP];
#pragma unroll
          for (int s = 0; s < PP; ++s) {
            pr[s] = 0.f;
            if (!active[s]) continue;                         // warp-uniform
            const int pos = pos_first + (warp + NWARP * s) / nh, lo = max(0, pos - a.window + 1);
            float sc = dot[s] * sc_mul;
            if (a.softcap > 0.f) sc = a.softcap * tanhf(sc / a.softcap);
            const int j = j0 + lane;
            if (lane >= nk || j < lo || j > pos) sc = -INFINITY;
            const float m_new = fmaxf(m_run[s], warp_max(sc));  // finite: at least one key of the stage is visible
            pr[s] = expf(sc - m_new);
            const float al = expf(m_run[s] - m_new);
            l_run[s] = l_run[s] * al + warp_sum(pr[s]);
            m_run[s] = m_new;
#pragma unroll
            for (int c = 0; c < VR; ++c) acc[s][c] *= al;
          }
          const float* vr = vs + gi * TK * a.vdim;
          const int jj_end = min(nk - 1, pos_max - j0);
          for (int jj = max(0, lo_min - j0); jj <= jj_end; ++jj) {
            float vv[VR];
#pragma unroll
            for (int c = 0; c < VR; ++c) {
              const int ch = lane + 32 * c;
              vv[c] = ch < a.vdim ? vr[jj * a.vdim + ch] : 0.f;
            }
#pragma unroll
            for (int s = 0; s < PP; ++s) {
              const float pw = __shfl_sync(0xffffffffu, pr[s], jj);   // 0 for a row that does not see key jj
#pragma unroll
              for (int c = 0; c < VR; ++c) acc[s][c] = fmaf(pw, vv[c], acc[s][c]);
            }
          }
        }
        continue;
      }
#pragma unroll
      for (int s = 0; s < PP; ++s) {
        const int p = warp + NWARP * s;
        if (p >= npairs) continue;
        const int i = p / nh, hh = p - i * nh;
        const int pos = pos_first + i, lo = max(0, pos - a.window + 1);
        if (j0 > pos || j0 + nk - 1 < lo) continue;          // no key of this stage is visible to the row (warp-uniform)
        const int h = h0 + hh, gi = h / rep - g_lo;
        const float* kr = ks + (gi * TK + lane) * DKS;
        const float* qr = qs + p * a.dim;
        float dot = 0.f;
        if (dot4) {
          const float4* k4 = reinterpret_cast<const float4*>(kr);
          const float4* q4 = reinterpret_cast<const float4*>(qr);
          for (int d = 0; d < a.dim / 4; ++d) {
            const float4 x = q4[d], y = k4[d];
            dot = fmaf(x.x, y.x, fmaf(x.y, y.y, fmaf(x.z, y.z, fmaf(x.w, y.w, dot))));
          }
        } else {
          for (int d = 0; d < a.dim; ++d) dot = fmaf(qr[d], kr[d], dot);
        }
        float sc = dot * a.scale * temp[h];
        if (a.softcap > 0.f) sc = a.softcap * tanhf(sc / a.softcap);
        const int j = j0 + lane;
        if (lane >= nk || j < lo || j > pos) sc = -INFINITY;
        const float m_new = fmaxf(m_run[s], warp_max(sc));      // finite: at least one key of the stage is visible
        const float pr = expf(sc - m_new);
        const float al = expf(m_run[s] - m_new);
        l_run[s] = l_run[s] * al + warp_sum(pr);
        m_run[s] = m_new;
#pragma unroll
        for (int c = 0; c < VR; ++c) acc[s][c] *= al;
        const float* vr = vs + gi * TK * a.vdim;
        const int jj_end = min(nk - 1, pos - j0);
        for (int jj = max(0, lo - j0); jj <= jj_end; ++jj) {
          const float pw = __shfl_sync(0xffffffffu, pr, jj);
#pragma unroll
          for (int c = 0; c < VR; ++c) {
            const int ch = lane + 32 * c;
            if (ch < a.vdim) acc[s][c] = fmaf(pw, vr[jj * a.vdim + ch], acc[s][c]);
          }
        }
      }
    }
#pragma unroll
    for (int s = 0; s < PP; ++s) {
      const int p = warp + NWARP * s;
      if (p >= npairs) continue;
      const int i = p / nh, hh = p - i * nh;
      const size_t rh = (size_t)(r + i) * a.H + h0 + hh;
      if (a.nsplit == 1) {
        const float invl = 1.0f / l_run[s];
#pragma unroll
        for (int c = 0; c < VR; ++c) {
          const int ch = lane + 32 * c;
          if (ch < a.vdim) stf(out + rh * a.vdim + ch, acc[s][c] * invl);
        }
      } else {
#pragma unroll
        for (int c = 0; c < VR; ++c) {
          const int ch = lane + 32 * c;
          if (ch < a.vdim) part[(rh * a.nsplit + z) * a.vdim + ch] = acc[s][c];
        }
        if (lane == 0) part_ml[rh * a.nsplit + z] = make_float2(m_run[s], l_run[s]);
      }
    }
    r = re;
  }
}

// out[rh] = sum_z part[rh][z] e^(m_z - m) / sum_z l_z e^(m_z - m), m = max_z m_z (a part without visible keys has m = -inf, l = 0)
template <typename T>
__global__ void __launch_bounds__(128) window_combine_kernel(const float* __restrict__ part, const float2* __restrict__ part_ml, T* __restrict__ out,
                                                             int vdim, int nsplit) {
  const size_t rh = blockIdx.x;
  float m = -INFINITY;
  for (int z = 0; z < nsplit; ++z) m = fmaxf(m, part_ml[rh * nsplit + z].x);
  float l = 0.f;
  for (int z = 0; z < nsplit; ++z) {
    const float2 ml = part_ml[rh * nsplit + z];
    if (ml.y > 0.f) l += ml.y * expf(ml.x - m);
  }
  const float invl = 1.0f / l;
  for (int c = threadIdx.x; c < vdim; c += 128) {
    float s = 0.f;
    for (int z = 0; z < nsplit; ++z) {
      const float2 ml = part_ml[rh * nsplit + z];
      if (ml.y > 0.f) s = fmaf(part[(rh * nsplit + z) * vdim + c], expf(ml.x - m), s);
    }
    stf(out + rh * vdim + c, s * invl);
  }
}

size_t attn_smem(const WindowArgs& a) {
  return ((size_t)(a.QR * a.HB * a.dim + 3) / 4 * 4 + (size_t)a.NG * TK * (key_stride(a.dim) + a.vdim)) * sizeof(float);
}

template <typename T, int VR, int PP>
int launch_attn(const void* q, int ldq, const void* kcache, long long kss, const void* vcache, long long vss, const int* meta, const float* temp,
                void* out, float* ws, int M, const WindowArgs& a, cudaStream_t stream) {
  LIA_CHECK_ARG((a.QR * a.HB + NWARP - 1) / NWARP <= PP, "lia_window_attn: %d rows x %d heads per block are too many for value heads of %d", a.QR, a.HB, a.vdim);
  const size_t smem = attn_smem(a);
  if (smem > 48 * 1024) LIA_CUDA(cudaFuncSetAttribute(window_attn_kernel<T, VR, PP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((M + a.QR - 1) / a.QR, (a.H + a.HB - 1) / a.HB, a.nsplit);
  float* part = ws;
  float2* part_ml = reinterpret_cast<float2*>(ws + (size_t)M * a.H * a.nsplit * a.vdim);
  window_attn_kernel<T, VR, PP><<<grid, NWARP * 32, smem, stream>>>(reinterpret_cast<const T*>(q), ldq, reinterpret_cast<const T*>(kcache), kss,
                                                                   reinterpret_cast<const T*>(vcache), vss, meta, temp, reinterpret_cast<T*>(out), part,
                                                                   part_ml, M, a);
  LIA_LAUNCH_CHECK();
  if (a.nsplit > 1) {
    window_combine_kernel<T><<<(unsigned)((size_t)M * a.H), 128, 0, stream>>>(part, part_ml, reinterpret_cast<T*>(out), a.vdim, a.nsplit);
    LIA_LAUNCH_CHECK();
  }
  return LIA_OK;
}

template <typename T>
int dispatch_attn(const void* q, int ldq, const void* kcache, long long kss, const void* vcache, long long vss, const int* meta, const float* temp,
                  void* out, float* ws, int M, const WindowArgs& a, cudaStream_t stream) {
  if (a.vdim <= 32) return launch_attn<T, 1, 4>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, ws, M, a, stream);
  if (a.vdim <= 64) return launch_attn<T, 2, 4>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, ws, M, a, stream);
  if (a.vdim <= 128) return launch_attn<T, 4, 4>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, ws, M, a, stream);
  if (a.vdim <= 256) return launch_attn<T, 8, 2>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, ws, M, a, stream);
  return launch_attn<T, 16, 1>(q, ldq, kcache, kss, vcache, vss, meta, temp, out, ws, M, a, stream);
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

// Pairs (row, head) that one warp can carry for value heads of `vdim` numbers: bounds rows_per_block * heads_per_block / 8.
extern "C" int lia_window_attn_pairs_per_warp(int vdim) { return vdim <= 128 ? 4 : (vdim <= 256 ? 2 : 1); }

extern "C" size_t lia_window_attn_smem_bytes(int heads_per_block, int kv_heads_per_block, int rows_per_block, int dim, int vdim) {
  WindowArgs a{0, 0, dim, vdim, 0, heads_per_block, kv_heads_per_block, rows_per_block, 1, 0.f, 0.f};
  return attn_smem(a);
}

extern "C" size_t lia_window_attn_workspace_floats(int M, int H, int vdim, int nsplit) {
  if (nsplit <= 1) return 0;
  return (size_t)M * H * nsplit * ((size_t)vdim + 2);
}

extern "C" int lia_window_attn(const void* q, int ldq, int act_f32, const void* kcache, long long k_slot_stride, const void* vcache,
                               long long v_slot_stride, const int* meta, const float* temp, void* out, float* workspace, int M, int H, int G,
                               int dim, int vdim, int window, float scale, float softcap, int heads_per_block, int rows_per_block, int nsplit,
                               lia_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LIA_CHECK_ARG(q && kcache && vcache && meta && temp && out, "lia_window_attn: null pointer");
  LIA_CHECK_ARG(M > 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && vdim <= 512 && window > 0 && H <= 65535 && ldq >= H * dim,
                "lia_window_attn: bad shape H=%d G=%d dim=%d vdim=%d window=%d", H, G, dim, vdim, window);
  const int rep = H / G, HB = heads_per_block;
  LIA_CHECK_ARG(HB >= 1 && HB <= NWARP && (HB % rep == 0 || rep % HB == 0), "lia_window_attn: %d heads per block do not fit groups of %d", HB, rep);
  LIA_CHECK_ARG(rows_per_block >= 1 && nsplit >= 1 && nsplit <= 64 && (nsplit == 1 || workspace), "lia_window_attn: bad rows per block (%d) or key ranges (%d)", rows_per_block, nsplit);
  WindowArgs a{H, G, dim, vdim, window, HB, HB >= rep ? HB / rep : 1, rows_per_block, nsplit, scale, softcap};
  LIA_CHECK_ARG(attn_smem(a) <= 200 * 1024, "lia_window_attn: heads of %d + %d numbers do not fit the shared-memory stage", dim, vdim);
  if (act_f32) return dispatch_attn<float>(q, ldq, kcache, k_slot_stride, vcache, v_slot_stride, meta, temp, out, workspace, M, a, stream);
  return dispatch_attn<bf16>(q, ldq, kcache, k_slot_stride, vcache, v_slot_stride, meta, temp, out, workspace, M, a, stream);
}
