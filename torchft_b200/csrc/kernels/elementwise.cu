// HBM-bound kernels of the Llama training step: embedding, RMSNorm (+ residual add),
// RoPE, SwiGLU, fused softmax cross-entropy, fused AdamW, gradient-norm.  All tensors
// are bf16 unless stated, rows are contiguous, and every row length must be a multiple
// of 8 elements so that all traffic is 16-byte vectors.
#include <algorithm>

#include "ftb200_common.cuh"

using ftb200::bf16x8;
using ftb200::pack8;
using ftb200::unpack8;

namespace {

// ------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ tok, const bf16x8* __restrict__ table,
                                     bf16x8* __restrict__ out, int T, int D8, int V) {
  const int t = blockIdx.x;
  if (t >= T) return;
  int64_t id = tok[t];
  if (!FTB_IN_RANGE(id, V) || id < 0 || id >= V) id = 0;  // an id outside the vocabulary reads row 0
  const bf16x8* src = table + id * D8;
  bf16x8* dst = out + static_cast<int64_t>(t) * D8;
  for (int i = threadIdx.x; i < D8; i += blockDim.x) dst[i] = src[i];
}

__global__ void embedding_bwd_kernel(const int64_t* __restrict__ tok, const __nv_bfloat162* __restrict__ dout,
                                     __nv_bfloat162* __restrict__ dtable, int T, int D2, int V) {
  const int t = blockIdx.x;
  if (t >= T) return;
  int64_t id = tok[t];
  if (!FTB_IN_RANGE(id, V) || id < 0 || id >= V) return;
  const __nv_bfloat162* src = dout + static_cast<int64_t>(t) * D2;
  __nv_bfloat162* dst = dtable + id * D2;
  for (int i = threadIdx.x; i < D2; i += blockDim.x) atomicAdd(dst + i, src[i]);
}

// ------------------------------------------------------------------ RMSNorm
// out = x * rstd * w ;  optionally first h = x + res (written to h_out) and normalise h.
__global__ void rmsnorm_fwd_kernel(const bf16x8* __restrict__ x, const bf16x8* __restrict__ res,
                                   bf16x8* __restrict__ h_out, const bf16x8* __restrict__ w,
                                   bf16x8* __restrict__ out, float* __restrict__ rstd_out, int D8, float eps) {
  __shared__ float scratch[33];
  const int64_t row = blockIdx.x;
  const bf16x8* xr = x + row * D8;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D8; i += blockDim.x) {
    float f[8];
    unpack8(xr[i], f);
    if (res != nullptr) {
      float g[8];
      unpack8(res[row * D8 + i], g);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] += g[e];
      bf16x8 hv = pack8(f);
      h_out[row * D8 + i] = hv;
      unpack8(hv, f);  // normalise the rounded value that later passes will read
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
  }
  ss = ftb200::block_sum(ss, scratch);
  const float r = rsqrtf(ss / (8.f * D8) + eps);
  if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[row] = r;
  if (out == nullptr) return;
  const bf16x8* src = (res != nullptr) ? (h_out + row * D8) : xr;
  for (int i = threadIdx.x; i < D8; i += blockDim.x) {
    float f[8], g[8];
    unpack8(src[i], f);
    unpack8(w[i], g);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = f[e] * r * g[e];
    out[row * D8 + i] = pack8(f);
  }
}

// dx = dres + rstd*w*dy - x*rstd^3/D * sum(dy*w*x);  dw partial sums per block.
// Each thread owns fixed 8-column groups so dw accumulates in registers across rows.
template <int MAXV>
__global__ void __launch_bounds__(512, MAXV == 1 ? 2 : 1) rmsnorm_bwd_kernel(const bf16x8* __restrict__ dy, const bf16x8* __restrict__ x,
                                   const bf16x8* __restrict__ w, const float* __restrict__ rstd,
                                   const bf16x8* __restrict__ dres, bf16x8* __restrict__ dx,
                                   float* __restrict__ dw_partial, int T, int D8) {
  __shared__ float scratch[66];
  float dw_acc[MAXV][8];
#pragma unroll
  for (int v = 0; v < MAXV; ++v)
#pragma unroll
    for (int e = 0; e < 8; ++e) dw_acc[v][e] = 0.f;

  // Two rows per iteration: their loads (dy, x and the residual gradient) are all in flight before the one
  // block-wide reduction they share, and the rows stay in registers (packed) across it.
  for (int64_t row0 = blockIdx.x; row0 < T; row0 += 2 * static_cast<int64_t>(gridDim.x)) {
    const int64_t rows[2] = {row0, row0 + gridDim.x};
    const bool live[2] = {true, rows[1] < T};
    float r[2] = {rstd[rows[0]], live[1] ? rstd[rows[1]] : 0.f};
    bf16x8 a[2][MAXV], b[2][MAXV], d[2][MAXV];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int i = threadIdx.x + v * blockDim.x;
        if (live[k] && i < D8) {
          a[k][v] = dy[rows[k] * D8 + i];
          b[k][v] = x[rows[k] * D8 + i];
          if (dres != nullptr) d[k][v] = dres[rows[k] * D8 + i];
        }
      }
    }
    float dot[2] = {0.f, 0.f};
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = threadIdx.x + v * blockDim.x;
      if (i < D8) {
        float c[8];
        unpack8(w[i], c);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          if (live[k]) {
            float fa[8], fb[8];
            unpack8(a[k][v], fa);
            unpack8(b[k][v], fb);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              dot[k] += fa[e] * c[e] * fb[e];
              dw_acc[v][e] += fa[e] * fb[e] * r[k];
            }
          }
        }
      }
    }
    const float2 dots = ftb200::block_sum2(dot[0], dot[1], scratch);
    const float coef[2] = {dots.x * r[0] * r[0] * r[0] / (8.f * D8), dots.y * r[1] * r[1] * r[1] / (8.f * D8)};
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = threadIdx.x + v * blockDim.x;
      if (i < D8) {
        float c[8];
        unpack8(w[i], c);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          if (live[k]) {
            float fa[8], fb[8], o[8];
            unpack8(a[k][v], fa);
            unpack8(b[k][v], fb);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = r[k] * c[e] * fa[e] - fb[e] * coef[k];
            if (dres != nullptr) {
              float fd[8];
              unpack8(d[k][v], fd);
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] += fd[e];
            }
            dx[rows[k] * D8 + i] = pack8(o);
          }
        }
      }
    }
  }
#pragma unroll
  for (int v = 0; v < MAXV; ++v) {
    const int i = threadIdx.x + v * blockDim.x;
    if (i < D8) {
      float* dst = dw_partial + (static_cast<int64_t>(blockIdx.x) * D8 + i) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) dst[e] = dw_acc[v][e];
    }
  }
}

// dw[c] (+)= sum_b partial[b][c].  A block owns 32 columns; its 8 warps stride over the rows (each warp
// instruction reads one 128-byte row segment) and meet in shared memory, so a few hundred rows are a few
// dozen independent loads per thread instead of one long serial loop.
__global__ void colsum_partials_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dw, int nblk, int D,
                                       int accumulate) {
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < D) {
#pragma unroll 4
    for (int b = ry; b < nblk; b += 8) s += partial[static_cast<int64_t>(b) * D + c];
  }
  red[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && c < D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][cx];
    if (accumulate) t += __bfloat162float(dw[c]);
    dw[c] = __float2bfloat16(t);
  }
}

// ------------------------------------------------------------------ RoPE (interleaved pairs)
// buf rows are [n_rot_heads * Dh | untouched tail]; cs = [S, Dh/2] of (cos, sin).
// One thread rotates 8 consecutive elements (4 pairs): one 16-byte load/store of data and
// two 16-byte loads of the table.
__global__ void rope_kernel(bf16x8* __restrict__ buf, const float4* __restrict__ cs, int64_t T, int S, int n_heads,
                            int Dh8, int64_t row_stride8, float sin_sign) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t per_row = static_cast<int64_t>(n_heads) * Dh8;
  if (idx >= T * per_row) return;
  const int64_t t = idx / per_row;
  const int r = static_cast<int>(idx - t * per_row);
  const int v = r % Dh8;  // which group of 4 pairs inside the head
  const int pos = static_cast<int>(t % S);
  const float4* c = cs + (static_cast<int64_t>(pos) * Dh8 + v) * 2;  // 4 (cos, sin) pairs = 2 float4
  const float4 c0 = c[0], c1 = c[1];
  const float cosv[4] = {c0.x, c0.z, c1.x, c1.z};
  const float sinv[4] = {c0.y * sin_sign, c0.w * sin_sign, c1.y * sin_sign, c1.w * sin_sign};
  if (!FTB_IN_RANGE(r, row_stride8)) return;  // rotated heads must fit inside a row
  bf16x8* p = buf + t * row_stride8 + r;
  float f[8];
  unpack8(*p, f);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float a = f[2 * e], b = f[2 * e + 1];
    f[2 * e] = a * cosv[e] - b * sinv[e];
    f[2 * e + 1] = a * sinv[e] + b * cosv[e];
  }
  *p = pack8(f);
}

// ------------------------------------------------------------------ SwiGLU
// gu rows hold interleaved (gate_j, up_j) pairs: [g0 u0 g1 u1 ...] (2F values);
// out[j] = silu(g_j) * u_j.  One thread handles 4 pairs.
__device__ __forceinline__ void store4_bf16(__nv_bfloat16* p, const float* f) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(f[0], f[1]), hi = __floats2bfloat162_rn(f[2], f[3]);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t*>(&lo);
  o.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = o;
}

__global__ void swiglu_fwd_kernel(const bf16x8* __restrict__ gu, __nv_bfloat16* __restrict__ out, int64_t n8) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= n8) return;
  float f[8], o[4];
  unpack8(gu[idx], f);
#pragma unroll
  for (int e = 0; e < 4; ++e) o[e] = f[2 * e] / (1.f + __expf(-f[2 * e])) * f[2 * e + 1];
  store4_bf16(out + idx * 4, o);
}

// dgu pair = (ds * u * dsilu(g), ds * silu(g))   (may alias gu: in place)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ ds, const bf16x8* gu, bf16x8* dgu, int64_t n8) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= n8) return;
  float f[8], o[8];
  unpack8(gu[idx], f);
  const uint2 raw = *reinterpret_cast<const uint2*>(ds + idx * 4);
  const float2 d01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 d23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  const float d[4] = {d01.x, d01.y, d23.x, d23.y};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float g = f[2 * e], u = f[2 * e + 1];
    const float sg = 1.f / (1.f + __expf(-g));
    const float silu = g * sg;
    o[2 * e] = d[e] * u * (sg + silu * (1.f - sg));
    o[2 * e + 1] = d[e] * silu;
  }
  dgu[idx] = pack8(o);
}

// ------------------------------------------------------------------ cross-entropy
// One block per row.  loss[row] = logsumexp(row) - row[target]; the row is overwritten
// in place by (softmax - onehot) * grad_scale.
__global__ void cross_entropy_kernel(bf16x8* __restrict__ logits, const int64_t* __restrict__ target,
                                     float* __restrict__ loss, int V8, int64_t ld8, float grad_scale) {
  __shared__ float scratch[33];
  const int64_t row = blockIdx.x;
  bf16x8* lr = logits + row * ld8;
  float mx = -INFINITY, sum = 0.f;
  for (int i = threadIdx.x; i < V8; i += blockDim.x) {
    float f[8];
    unpack8(lr[i], f);
    float cm = f[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) cm = fmaxf(cm, f[e]);
    if (cm > mx) {
      sum *= __expf(mx - cm);
      mx = cm;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) sum += __expf(f[e] - mx);
  }
  const float gmx = ftb200::block_max(mx, scratch);
  sum *= __expf(mx - gmx);
  const float gsum = ftb200::block_sum(sum, scratch);
  const int64_t tgt = target[row];
  if (tgt >= 0) (void)FTB_IN_RANGE(tgt, 8 * static_cast<int64_t>(V8));  // negative targets mean "ignore"
  (void)FTB_IN_RANGE(V8 - 1, ld8);                                        // a row must fit inside its stride
  const float inv = 1.f / gsum;
  if (threadIdx.x == 0) {
    const __nv_bfloat16* flat = reinterpret_cast<const __nv_bfloat16*>(lr);
    const float xt = (tgt >= 0 && tgt < 8 * static_cast<int64_t>(V8)) ? __bfloat162float(flat[tgt]) : 0.f;
    loss[row] = (tgt >= 0) ? (logf(gsum) + gmx - xt) : 0.f;
  }
  __syncthreads();  // the target logit is read before any thread overwrites it
  const float gs = (tgt >= 0) ? grad_scale : 0.f;
  for (int i = threadIdx.x; i < V8; i += blockDim.x) {
    float f[8];
    unpack8(lr[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float pr = __expf(f[e] - gmx) * inv;
      if (static_cast<int64_t>(i) * 8 + e == tgt) pr -= 1.f;
      f[e] = pr * gs;
    }
    lr[i] = pack8(f);
  }
}

// ------------------------------------------------------------------ AdamW (flat shard)
// master/m/v fp32, grad bf16 or fp32, writes the bf16 working copy.  `grad_scale_dev`
// (optional) is a device scalar multiplied into every gradient (clipping coefficient).
template <typename G>
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16, int64_t n, float lr,
                             float beta1, float beta2, float eps, float wd, float bc1, float bc2_sqrt,
                             const float* __restrict__ grad_scale_dev) {
  const float gs = grad_scale_dev ? *grad_scale_dev : 1.f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * 4;
  for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 p4 = *reinterpret_cast<float4*>(master + i);
      float4 m4 = *reinterpret_cast<float4*>(m + i);
      float4 v4 = *reinterpret_cast<float4*>(v + i);
      float g[4];
      if constexpr (sizeof(G) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(grad + i);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
      } else {
        const float4 gg = *reinterpret_cast<const float4*>(grad + i);
        g[0] = gg.x; g[1] = gg.y; g[2] = gg.z; g[3] = gg.w;
      }
      float* pp = &p4.x;
      float* mm = &m4.x;
      float* vv = &v4.x;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float ge = g[e] * gs;
        mm[e] = beta1 * mm[e] + (1.f - beta1) * ge;
        vv[e] = beta2 * vv[e] + (1.f - beta2) * ge * ge;
        const float denom = sqrtf(vv[e]) / bc2_sqrt + eps;
        pp[e] = pp[e] * (1.f - lr * wd) - (lr / bc1) * (mm[e] / denom);
      }
      *reinterpret_cast<float4*>(master + i) = p4;
      *reinterpret_cast<float4*>(m + i) = m4;
      *reinterpret_cast<float4*>(v + i) = v4;
      if (param_bf16 != nullptr) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(p4.x, p4.y), hi = __floats2bfloat162_rn(p4.z, p4.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(param_bf16 + i) = o;
      }
    } else {
      for (int64_t j = i; j < n; ++j) {
        float ge;
        if constexpr (sizeof(G) == 2) ge = __bfloat162float(grad[j]) * gs; else ge = grad[j] * gs;
        const float mj = beta1 * m[j] + (1.f - beta1) * ge;
        const float vj = beta2 * v[j] + (1.f - beta2) * ge * ge;
        const float denom = sqrtf(vj) / bc2_sqrt + eps;
        const float pj = master[j] * (1.f - lr * wd) - (lr / bc1) * (mj / denom);
        m[j] = mj; v[j] = vj; master[j] = pj;
        if (param_bf16 != nullptr) param_bf16[j] = __float2bfloat16(pj);
      }
    }
  }
}

// sum of squares of a bf16 (or fp32) buffer, accumulated into *out with one atomic per block.
template <typename G>
__global__ void sumsq_kernel(const G* __restrict__ x, int64_t n, float* __restrict__ out) {
  __shared__ float scratch[33];
  float s = 0.f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if constexpr (sizeof(G) == 2) {
    const int64_t n8 = n / 8;
    const bf16x8* xv = reinterpret_cast<const bf16x8*>(x);
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
      float f[8];
      unpack8(xv[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) s += f[e] * f[e];
    }
    for (int64_t j = n8 * 8 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride) {
      const float f = __bfloat162float(x[j]);
      s += f * f;
    }
  } else {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) s += x[i] * x[i];
  }
  s = ftb200::block_sum(s, scratch);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// coef = min(1, max_norm / (sqrt(sumsq) + 1e-6)); also stores the norm.
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm, float* __restrict__ coef,
                                 float* __restrict__ norm_out) {
  const float nrm = sqrtf(*sumsq);
  if (norm_out) *norm_out = nrm;
  *coef = (max_norm > 0.f) ? fminf(1.f, max_norm / (nrm + 1e-6f)) : 1.f;
}

int grid_for(int64_t work_items, int block) {
  int64_t g = (work_items + block - 1) / block;
  return static_cast<int>(g < 1 ? 1 : g);
}

}  // namespace

FTB200_API int ftb200_embedding_fwd(const int64_t* tok, const void* table, void* out, int T, int D, int V,
                                    cudaStream_t st) {
  if (D % 8) return FTB200_E_ALIGN;
  embedding_fwd_kernel<<<T, 256, 0, st>>>(tok, (const bf16x8*)table, (bf16x8*)out, T, D / 8, V);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_embedding_bwd(const int64_t* tok, const void* dout, void* dtable, int T, int D, int V,
                                    cudaStream_t st) {
  if (D % 8) return FTB200_E_ALIGN;
  embedding_bwd_kernel<<<T, 256, 0, st>>>(tok, (const __nv_bfloat162*)dout, (__nv_bfloat162*)dtable, T, D / 2, V);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// res/h_out may be null (plain norm); out may be null (only rstd wanted).
FTB200_API int ftb200_rmsnorm_fwd(const void* x, const void* res, void* h_out, const void* w, void* out, float* rstd,
                                  int T, int D, float eps, cudaStream_t st) {
  if (D % 8) return FTB200_E_ALIGN;
  if (res != nullptr && h_out == nullptr) return FTB200_E_BADARG;
  const int threads = (D / 8 >= 512) ? 512 : 256;
  rmsnorm_fwd_kernel<<<T, threads, 0, st>>>((const bf16x8*)x, (const bf16x8*)res, (bf16x8*)h_out, (const bf16x8*)w,
                                            (bf16x8*)out, rstd, D / 8, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// Number of floats the caller must provide in `dw_partial` for ftb200_rmsnorm_bwd.
FTB200_API long long ftb200_rmsnorm_bwd_scratch_floats(int D) {
  return static_cast<long long>(ftb200::sm_count()) * 2 * D;
}

FTB200_API int ftb200_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                  void* dx, void* dw, float* dw_partial, int T, int D, int accumulate_dw,
                                  cudaStream_t st) {
  if (D % 8) return FTB200_E_ALIGN;
  const int D8 = D / 8;
  const int threads = D8 > 256 ? 512 : 256;  // wide rows: 16 warps per block, two blocks per SM
  const int nblk = min(T, ftb200::sm_count() * 2);
  const int maxv = (D8 + threads - 1) / threads;
  if (maxv <= 1)
    rmsnorm_bwd_kernel<1><<<nblk, threads, 0, st>>>((const bf16x8*)dy, (const bf16x8*)x, (const bf16x8*)w, rstd,
                                                    (const bf16x8*)dres, (bf16x8*)dx, dw_partial, T, D8);
  else if (maxv <= 2)
    rmsnorm_bwd_kernel<2><<<nblk, threads, 0, st>>>((const bf16x8*)dy, (const bf16x8*)x, (const bf16x8*)w, rstd,
                                                    (const bf16x8*)dres, (bf16x8*)dx, dw_partial, T, D8);
  else if (maxv <= 4)
    rmsnorm_bwd_kernel<4><<<nblk, threads, 0, st>>>((const bf16x8*)dy, (const bf16x8*)x, (const bf16x8*)w, rstd,
                                                    (const bf16x8*)dres, (bf16x8*)dx, dw_partial, T, D8);
  else
    return FTB200_E_TOOBIG;  // D > 8192
  colsum_partials_kernel<<<(D + 31) / 32, 256, 0, st>>>(dw_partial, (__nv_bfloat16*)dw, nblk, D, accumulate_dw);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// Rotates the first n_heads heads of every row in place.  backward != 0 applies the inverse rotation.
FTB200_API int ftb200_rope(void* buf, const float* cos_sin, long long T, int S, int n_heads, int head_dim,
                           long long row_stride, int backward, cudaStream_t st) {
  if (head_dim % 8 || row_stride % 8 || (reinterpret_cast<uintptr_t>(buf) & 15)) return FTB200_E_ALIGN;
  const int64_t total = T * n_heads * (head_dim / 8);
  rope_kernel<<<grid_for(total, 256), 256, 0, st>>>((bf16x8*)buf, (const float4*)cos_sin, T, S, n_heads, head_dim / 8,
                                                    row_stride / 8, backward ? -1.f : 1.f);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_swiglu_fwd(const void* gu, void* out, long long T, int F, cudaStream_t st) {
  if (F % 4) return FTB200_E_ALIGN;
  const int64_t n8 = T * (F / 4);
  swiglu_fwd_kernel<<<grid_for(n8, 256), 256, 0, st>>>((const bf16x8*)gu, (__nv_bfloat16*)out, n8);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_swiglu_bwd(const void* ds, const void* gu, void* dgu, long long T, int F, cudaStream_t st) {
  if (F % 4) return FTB200_E_ALIGN;
  const int64_t n8 = T * (F / 4);
  swiglu_bwd_kernel<<<grid_for(n8, 256), 256, 0, st>>>((const __nv_bfloat16*)ds, (const bf16x8*)gu, (bf16x8*)dgu, n8);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_cross_entropy(void* logits, const int64_t* target, float* loss, int T, int V, long long ld,
                                    float grad_scale, cudaStream_t st) {
  if (V % 8 || ld % 8) return FTB200_E_ALIGN;
  cross_entropy_kernel<<<T, 1024, 0, st>>>((bf16x8*)logits, target, loss, V / 8, ld / 8, grad_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_adamw(float* master, float* m, float* v, const void* grad, int grad_is_fp32, void* param_bf16,
                            long long n, float lr, float beta1, float beta2, float eps, float wd, int step,
                            const float* grad_scale_dev, cudaStream_t st) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15)
    return FTB200_E_ALIGN;
  if (reinterpret_cast<uintptr_t>(grad) & (grad_is_fp32 ? 15 : 7)) return FTB200_E_ALIGN;
  if (reinterpret_cast<uintptr_t>(param_bf16) & 7) return FTB200_E_ALIGN;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2s = sqrtf(1.f - powf(beta2, static_cast<float>(step)));
  const int blocks = static_cast<int>(std::min<long long>((n / 4 + 255) / 256 + 1, ftb200::sm_count() * 16LL));
  if (grad_is_fp32)
    adamw_kernel<float><<<blocks, 256, 0, st>>>(master, m, v, (const float*)grad, (__nv_bfloat16*)param_bf16, n, lr,
                                                beta1, beta2, eps, wd, bc1, bc2s, grad_scale_dev);
  else
    adamw_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(master, m, v, (const __nv_bfloat16*)grad,
                                                        (__nv_bfloat16*)param_bf16, n, lr, beta1, beta2, eps, wd, bc1,
                                                        bc2s, grad_scale_dev);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// *out += sum(x^2).  The caller zeroes *out before the first call of a step.
FTB200_API int ftb200_sumsq(const void* x, int is_fp32, long long n, float* out, cudaStream_t st) {
  if (n <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(x) & 15) return FTB200_E_ALIGN;
  const int blocks = static_cast<int>(std::min<long long>((n / 8 + 255) / 256 + 1, ftb200::sm_count() * 8LL));
  if (is_fp32)
    sumsq_kernel<float><<<blocks, 256, 0, st>>>((const float*)x, n, out);
  else
    sumsq_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, n, out);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_clip_coef(const float* sumsq, float max_norm, float* coef, float* norm_out, cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>(sumsq, max_norm, coef, norm_out);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// ------------------------------------------------------------------ allocation-free variant
// See ftb200_noalloc.h.  The scratch lives in the library image; host code must not pass
// the symbol itself to a kernel (on the host it is only a stand-in), so its device address
// is looked up once per device and cached.
#include <atomic>

#include "ftb200_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[FTB200_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
// Host threads may make their first call on a device at the same time: they all resolve the
// same address, and the atomic makes the concurrent store and loads well defined.
std::atomic<float*> g_noalloc_scratch_addr[kMaxDevices];
}  // namespace

FTB200_API int ftb200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                          const void* dres, void* dx, void* dw, int T, int D, int accumulate_dw,
                                          cudaStream_t st) {
  if (T <= 0 || D <= 0 || dy == nullptr || x == nullptr || w == nullptr || rstd == nullptr || dx == nullptr ||
      dw == nullptr)
    return FTB200_E_BADARG;
  if (D % 8) return FTB200_E_ALIGN;
  if (D > 8192) return FTB200_E_TOOBIG;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FTB200_E_CUDA;
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return FTB200_E_CUDA;
  const int nblk = std::min(T, sms * 2);
  if (static_cast<long long>(nblk) * D > static_cast<long long>(FTB200_NOALLOC_SCRATCH_FLOATS)) return FTB200_E_TOOBIG;
  float* scratch = g_noalloc_scratch_addr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // one-time set-up for this device (which is current): resolve the array's device address
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return FTB200_E_CUDA;
    }
    g_noalloc_scratch_addr[dev].store(p, std::memory_order_release);
    scratch = p;
  }
  const int D8 = D / 8;
  const int threads = D8 > 256 ? 512 : 256;  // wide rows: 16 warps per block, two blocks per SM
  const int maxv = (D8 + threads - 1) / threads;
  if (maxv <= 1)
    rmsnorm_bwd_kernel<1><<<nblk, threads, 0, st>>>((const bf16x8*)dy, (const bf16x8*)x, (const bf16x8*)w, rstd,
                                                    (const bf16x8*)dres, (bf16x8*)dx, scratch, T, D8);
  else if (maxv <= 2)
    rmsnorm_bwd_kernel<2><<<nblk, threads, 0, st>>>((const bf16x8*)dy, (const bf16x8*)x, (const bf16x8*)w, rstd,
                                                    (const bf16x8*)dres, (bf16x8*)dx, scratch, T, D8);
  else
    rmsnorm_bwd_kernel<4><<<nblk, threads, 0, st>>>((const bf16x8*)dy, (const bf16x8*)x, (const bf16x8*)w, rstd,
                                                    (const bf16x8*)dres, (bf16x8*)dx, scratch, T, D8);
  colsum_partials_kernel<<<(D + 31) / 32, 256, 0, st>>>(scratch, (__nv_bfloat16*)dw, nblk, D, accumulate_dw);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// ---- checked-index debug build: status query and a self-test that records an out-of-range
// index without touching memory (a launch of one thread evaluating FTB_IN_RANGE(5, 4))
#ifdef FT_BOUNDS_CHECK
namespace {
__global__ void bounds_selftest_kernel(int i, int n, int* ok) { *ok = FTB_IN_RANGE(i, n) ? 1 : 0; }
}  // namespace
FTB200_API int ftb200_bounds_selftest(int i, int n, int* ok_dev, cudaStream_t st) {
  bounds_selftest_kernel<<<1, 1, 0, st>>>(i, n, ok_dev);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}
#endif
FTB_DEFINE_BOUNDS_QUERY(elementwise)
