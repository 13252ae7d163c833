// Bandwidth-bound ops for sm_100a: RMSNorm / LayerNorm (fwd + bwd), GELU, SwiGLU, RoPE, column sums,
// embedding gather / scatter-add, cross-entropy (fwd + bwd) and fused AdamW.  Everything moves 16-byte
// vectors, keeps a row in registers between the statistics pass and the normalisation pass (one read of
// x per op), and does its arithmetic in fp32.  Grids are sized from the SM count (persistent row loops)
// so that a launch is one wave.
#include "common.cuh"

namespace jpb {

template <typename T> struct Vec;  // 16-byte vector of T
template <> struct Vec<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = raw; }
  __device__ __forceinline__ void to_float(float (&f)[4]) const { f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w; }
  __device__ __forceinline__ void from_float(const float (&f)[4]) { raw = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ void to_float(float (&f)[8]) const {
    float2 a = unpack_bf16(raw.x), b = unpack_bf16(raw.y), c = unpack_bf16(raw.z), d = unpack_bf16(raw.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  __device__ __forceinline__ void from_float(const float (&f)[8]) {
    raw.x = pack_bf16(f[0], f[1]); raw.y = pack_bf16(f[2], f[3]); raw.z = pack_bf16(f[4], f[5]); raw.w = pack_bf16(f[6], f[7]);
  }
};

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Sum (and optionally a second sum) over a CTA; result broadcast to all threads.
template <int NV>
__device__ __forceinline__ void block_sum(float (&v)[NV], float* scratch /* >= NV*32 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int i = 0; i < NV; ++i) v[i] = warp_sum(v[i]);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i) scratch[i * 32 + warp] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float x = lane < nwarps ? scratch[i * 32 + lane] : 0.f;
    v[i] = warp_sum(x);
  }
}

constexpr int NORM_MAX_VECS = 4;  // vectors per thread kept in registers (forward)
constexpr int NORM_BWD_VECS = 2;  // backward keeps more state per vector

// ---------------------------------------------------------------------------------------------------------
// RMSNorm / LayerNorm forward.  One CTA per row (grid-stride), blockDim = ceil(H / VEC / vecs_per_thread).
// ---------------------------------------------------------------------------------------------------------
template <typename T, bool LAYER>
__global__ void norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                                int H, float eps) {
  constexpr int VN = Vec<T>::N;
  __shared__ float scratch[64];
  const int nvec = H / VN;
  // the next row is requested before this row's block reduction, so that loads stay in flight across the barriers
  // and the stores (a CTA that loads, reduces and stores one row at a time keeps the memory system busy about a
  // third of the time)
  Vec<T> xv[NORM_MAX_VECS], xn[NORM_MAX_VECS];
  if (blockIdx.x < rows) {
#pragma unroll
    for (int i = 0; i < NORM_MAX_VECS; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) xv[i].load(x + size_t(blockIdx.x) * H + v * VN);
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float s[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NORM_MAX_VECS; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float f[VN];
        xv[i].to_float(f);
#pragma unroll
        for (int j = 0; j < VN; ++j) { s[0] += f[j]; s[1] += f[j] * f[j]; }
      }
    }
    const int next = row + gridDim.x;
    if (next < rows) {
#pragma unroll
      for (int i = 0; i < NORM_MAX_VECS; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) xn[i].load(x + size_t(next) * H + v * VN);
      }
    }
    block_sum<2>(s, scratch);
    float mean = 0.f, rstd;
    if (LAYER) {
      mean = s[0] / H;
      // two-pass variance from registers for accuracy
      float q[1] = {0.f};
#pragma unroll
      for (int i = 0; i < NORM_MAX_VECS; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
          float f[VN];
          xv[i].to_float(f);
#pragma unroll
          for (int j = 0; j < VN; ++j) { const float d = f[j] - mean; q[0] += d * d; }
        }
      }
      block_sum<1>(q, scratch);
      rstd = rsqrtf(q[0] / H + eps);
    } else {
      rstd = rsqrtf(s[1] / H + eps);
    }
    if (threadIdx.x == 0) {
      rstd_out[row] = rstd;
      if (LAYER) mean_out[row] = mean;
    }
    T* yr = y + size_t(row) * H;
#pragma unroll
    for (int i = 0; i < NORM_MAX_VECS; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float f[VN], wf[VN], bf[VN];
        xv[i].to_float(f);
        Vec<T> wv; wv.load(w + v * VN); wv.to_float(wf);
        if (LAYER) { Vec<T> bv; bv.load(b + v * VN); bv.to_float(bf); }
#pragma unroll
        for (int j = 0; j < VN; ++j) f[j] = (f[j] - mean) * rstd * wf[j] + (LAYER ? bf[j] : 0.f);
        Vec<T> o; o.from_float(f); o.store(yr + v * VN);
      }
    }
#pragma unroll
    for (int i = 0; i < NORM_MAX_VECS; ++i) xv[i] = xn[i];
  }
}

// ---------------------------------------------------------------------------------------------------------
// RMSNorm / LayerNorm backward.  Each CTA walks rows (grid-stride), writes dx and keeps per-column partial
// sums of dw (and db) in registers; partials go to `partial[gridDim.x][2][H]` (scratch) and a second kernel
// reduces them.
// ---------------------------------------------------------------------------------------------------------
// MAXT = largest block the instantiation is launched with: 512 leaves room (128 registers per thread) for the
// next-row prefetch; the 1024-thread variant (very long rows) reloads each row after the barrier instead.
template <typename T, bool LAYER, int MAXT = 512>
__global__ void __launch_bounds__(MAXT) norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                T* __restrict__ dx, float* __restrict__ partial, int rows, int H,
                                const T* __restrict__ add = nullptr) {
  // `add` (optional, same shape as dx): the gradient arriving over the residual connection; dx_out = dx + add
  // with dx rounded to the storage type first, i.e. exactly what a separate add kernel would have produced.
  constexpr int VN = Vec<T>::N;
  __shared__ float scratch[64];
  const int nvec = H / VN;
  float dw_acc[NORM_BWD_VECS][VN], db_acc[NORM_BWD_VECS][VN];
#pragma unroll
  for (int i = 0; i < NORM_BWD_VECS; ++i)
#pragma unroll
    for (int j = 0; j < VN; ++j) { dw_acc[i][j] = 0.f; db_acc[i][j] = 0.f; }
  float wf[NORM_BWD_VECS][VN];
#pragma unroll
  for (int i = 0; i < NORM_BWD_VECS; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) { Vec<T> wv; wv.load(w + v * VN); wv.to_float(wf[i]); }
  }
  // the next row's x and dy are requested before this row's block reduction, so that loads stay in flight
  // across the barrier
  constexpr bool PREFETCH = MAXT <= 512;
  Vec<T> xv[NORM_BWD_VECS], dv[NORM_BWD_VECS];
  if (PREFETCH && blockIdx.x < rows) {
#pragma unroll
    for (int i = 0; i < NORM_BWD_VECS; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        xv[i].load(x + size_t(blockIdx.x) * H + v * VN);
        dv[i].load(dy + size_t(blockIdx.x) * H + v * VN);
      }
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    const float mean = LAYER ? mean_in[row] : 0.f;
    float xh[NORM_BWD_VECS][VN], g[NORM_BWD_VECS][VN];
    float s[2] = {0.f, 0.f};  // sum g, sum g*xhat
#pragma unroll
    for (int i = 0; i < NORM_BWD_VECS; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        if (!PREFETCH) {
          xv[i].load(x + size_t(row) * H + v * VN);
          dv[i].load(dy + size_t(row) * H + v * VN);
        }
        float xf[VN], df[VN];
        xv[i].to_float(xf); dv[i].to_float(df);
#pragma unroll
        for (int j = 0; j < VN; ++j) {
          xh[i][j] = (xf[j] - mean) * rstd;
          g[i][j] = df[j] * wf[i][j];
          s[0] += g[i][j];
          s[1] += g[i][j] * xh[i][j];
          dw_acc[i][j] += df[j] * xh[i][j];
          db_acc[i][j] += df[j];
        }
      }
    }
    const int next = row + gridDim.x;
    if (PREFETCH && next < rows) {
#pragma unroll
      for (int i = 0; i < NORM_BWD_VECS; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
          xv[i].load(x + size_t(next) * H + v * VN);
          dv[i].load(dy + size_t(next) * H + v * VN);
        }
      }
    }
    Vec<T> av[NORM_BWD_VECS];   // this row of `add`: requested before the barrier too
    if (add != nullptr) {
#pragma unroll
      for (int i = 0; i < NORM_BWD_VECS; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) av[i].load(add + size_t(row) * H + v * VN);
      }
    }
    block_sum<2>(s, scratch);
    const float m_g = LAYER ? s[0] / H : 0.f;
    const float m_gx = s[1] / H;
#pragma unroll
    for (int i = 0; i < NORM_BWD_VECS; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float o[VN];
#pragma unroll
        for (int j = 0; j < VN; ++j) o[j] = (g[i][j] - m_g - xh[i][j] * m_gx) * rstd;
        Vec<T> ov; ov.from_float(o);
        if (add != nullptr) {
          float r[VN], a[VN];
          ov.to_float(r); av[i].to_float(a);
#pragma unroll
          for (int j = 0; j < VN; ++j) r[j] = __fadd_rn(r[j], a[j]);  // never contracted into the multiply above
          ov.from_float(r);
        }
        ov.store(dx + size_t(row) * H + v * VN);
      }
    }
  }
  float* pw = partial + size_t(blockIdx.x) * 2 * H;
  float* pb = pw + H;
#pragma unroll
  for (int i = 0; i < NORM_BWD_VECS; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        pw[v * VN + j] = dw_acc[i][j];
        if (LAYER) pb[v * VN + j] = db_acc[i][j];
      }
    }
  }
}

// out[c] = sum_p partial[p * stride + c]   (p < nparts).  A CTA of 256 threads owns 32 columns: thread (cx, ry) adds up
// rows ry, ry + 8, ... of column cx (four independent loads in flight, 128 contiguous bytes per warp and row), and the
// eight row slices meet in shared memory.  One thread per column walking all rows, the earlier form, took as long as
// half the norm-backward kernel that produces the partial sums.
template <typename T>
__global__ void reduce_partials_kernel(const float* __restrict__ partial, T* __restrict__ out, int nparts, int cols,
                                       size_t stride) {
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  if (c < cols) {
    int p = ry;
    for (; p + 24 < nparts; p += 32) {
      a0 += partial[size_t(p) * stride + c];
      a1 += partial[size_t(p + 8) * stride + c];
      a2 += partial[size_t(p + 16) * stride + c];
      a3 += partial[size_t(p + 24) * stride + c];
    }
    for (; p < nparts; p += 8) a0 += partial[size_t(p) * stride + c];
  }
  red[ry][cx] = (a0 + a1) + (a2 + a3);
  __syncthreads();
  if (ry == 0 && c < cols) {
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += red[i][cx];
    out[c] = from_f<T>(acc);
  }
}

// ---------------------------------------------------------------------------------------------------------
// column sums of a [rows, cols] matrix into partial[gridDim.y][cols]
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void colsum_partial_kernel(const T* __restrict__ x, float* __restrict__ partial, int rows, int cols) {
  constexpr int VN = Vec<T>::N;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;  // vector column
  if (v * VN >= cols) return;
  float acc[VN];
#pragma unroll
  for (int j = 0; j < VN; ++j) acc[j] = 0.f;
  int r = blockIdx.y;
  for (; r + 3 * int(gridDim.y) < rows; r += 4 * gridDim.y) {   // four rows in flight per thread
    Vec<T> x0, x1, x2, x3;
    x0.load(x + size_t(r) * cols + v * VN);
    x1.load(x + size_t(r + gridDim.y) * cols + v * VN);
    x2.load(x + size_t(r + 2 * gridDim.y) * cols + v * VN);
    x3.load(x + size_t(r + 3 * gridDim.y) * cols + v * VN);
    float f0[VN], f1[VN], f2[VN], f3[VN];
    x0.to_float(f0); x1.to_float(f1); x2.to_float(f2); x3.to_float(f3);
#pragma unroll
    for (int j = 0; j < VN; ++j) acc[j] += (f0[j] + f1[j]) + (f2[j] + f3[j]);
  }
  for (; r < rows; r += gridDim.y) {
    Vec<T> xv; xv.load(x + size_t(r) * cols + v * VN);
    float f[VN]; xv.to_float(f);
#pragma unroll
    for (int j = 0; j < VN; ++j) acc[j] += f[j];
  }
#pragma unroll
  for (int j = 0; j < VN; ++j) partial[size_t(blockIdx.y) * cols + v * VN + j] = acc[j];
}

// ---------------------------------------------------------------------------------------------------------
// elementwise: GELU (tanh form), SwiGLU on [gate | up]
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanhf(k0 * (x + k1 * x * x * x));
  const float dt = (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
  return 0.5f * (1.f + t) + 0.5f * x * dt;
}

template <typename T, bool BWD>
__global__ void gelu_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ out, size_t nvec) {
  constexpr int VN = Vec<T>::N;
  for (size_t v = size_t(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += size_t(gridDim.x) * blockDim.x) {
    Vec<T> xv; xv.load(x + v * VN);
    float f[VN]; xv.to_float(f);
    if (BWD) {
      Vec<T> dv; dv.load(dy + v * VN);
      float d[VN]; dv.to_float(d);
#pragma unroll
      for (int j = 0; j < VN; ++j) f[j] = d[j] * gelu_grad_f(f[j]);
    } else {
#pragma unroll
      for (int j = 0; j < VN; ++j) f[j] = gelu_f(f[j]);
    }
    Vec<T> o; o.from_float(f); o.store(out + v * VN);
  }
}

// gate_up: [rows, 2F] (gate first); out: [rows, F]
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ out, size_t rows, int F) {
  constexpr int VN = Vec<T>::N;
  const int fv = F / VN;
  const size_t total = rows * fv;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t r = i / fv;
    const int c = int(i % fv) * VN;
    Vec<T> gv, uv;
    gv.load(gu + r * 2 * F + c);
    uv.load(gu + r * 2 * F + F + c);
    float g[VN], u[VN];
    gv.to_float(g); uv.to_float(u);
#pragma unroll
    for (int j = 0; j < VN; ++j) g[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    Vec<T> o; o.from_float(g); o.store(out + r * F + c);
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ gu, T* __restrict__ dgu, size_t rows,
                                  int F) {
  constexpr int VN = Vec<T>::N;
  const int fv = F / VN;
  const size_t total = rows * fv;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t r = i / fv;
    const int c = int(i % fv) * VN;
    Vec<T> gv, uv, dv;
    gv.load(gu + r * 2 * F + c);
    uv.load(gu + r * 2 * F + F + c);
    dv.load(dy + r * F + c);
    float g[VN], u[VN], d[VN], dg[VN], du[VN];
    gv.to_float(g); uv.to_float(u); dv.to_float(d);
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      dg[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
      du[j] = d[j] * g[j] * s;
    }
    Vec<T> og, ou;
    og.from_float(dg); ou.from_float(du);
    og.store(dgu + r * 2 * F + c);
    ou.store(dgu + r * 2 * F + F + c);
  }
}

// ---------------------------------------------------------------------------------------------------------
// RoPE, half-split convention: x[B,S,H,D]; cos/sin [S, D/2] fp32; inverse rotates by -theta
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                            T* __restrict__ out, size_t n_heads_total /* B*S*H */, int S, int H, int D, int inverse) {
  constexpr int VN = Vec<T>::N;
  const int hv = (D / 2) / VN;  // vectors per half
  const size_t total = n_heads_total * hv;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t head = i / hv;
    const int c = int(i % hv) * VN;
    const int s = int((head / H) % S);
    const T* xp = x + head * D;
    Vec<T> a, b;
    a.load(xp + c);
    b.load(xp + D / 2 + c);
    float af[VN], bf[VN], o1[VN], o2[VN];
    a.to_float(af); b.to_float(bf);
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      const float cc = cs[size_t(s) * (D / 2) + c + j];
      float ss = sn[size_t(s) * (D / 2) + c + j];
      if (inverse) ss = -ss;
      o1[j] = af[j] * cc - bf[j] * ss;
      o2[j] = bf[j] * cc + af[j] * ss;
    }
    Vec<T> v1, v2;
    v1.from_float(o1); v2.from_float(o2);
    v1.store(out + head * D + c);
    v2.store(out + head * D + D / 2 + c);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Fused split of a packed projection [rows, Hq + 2*Hkv, D] into contiguous q / k / v with RoPE applied to q
// and k on the way (cs == nullptr: plain split), and its transpose: merge dq / dk / dv into the packed
// gradient with the inverse rotation.  One pass over the data instead of three strided copies and two
// rotations (forward) or three zero fills, three copies, two adds and two rotations (backward).
// ---------------------------------------------------------------------------------------------------------
template <typename T, bool MERGE>
__global__ void qkv_rope_kernel(T* __restrict__ packed, T* __restrict__ q, T* __restrict__ k, T* __restrict__ v,
                                const float* __restrict__ cs, const float* __restrict__ sn, size_t rows, int S, int Hq,
                                int Hkv, int D) {
  constexpr int VN = Vec<T>::N;
  const int hv = (D / 2) / VN;
  const int Ht = Hq + 2 * Hkv;
  const size_t total = rows * Ht * hv;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t head = i / hv;
    const int c = int(i % hv) * VN;
    const size_t row = head / Ht;
    const int h = int(head % Ht);
    const int s = int(row % S);
    T* pp = packed + head * D;
    T* sp;
    bool rot = cs != nullptr;
    if (h < Hq) sp = q + (row * Hq + h) * D;
    else if (h < Hq + Hkv) sp = k + (row * Hkv + (h - Hq)) * D;
    else { sp = v + (row * Hkv + (h - Hq - Hkv)) * D; rot = false; }
    const T* src = MERGE ? sp : pp;
    T* dst = MERGE ? pp : sp;
    Vec<T> a, b;
    a.load(src + c);
    b.load(src + D / 2 + c);
    if (rot) {
      float af[VN], bf[VN], o1[VN], o2[VN];
      a.to_float(af); b.to_float(bf);
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        const float cc = cs[size_t(s) * (D / 2) + c + j];
        float ss = sn[size_t(s) * (D / 2) + c + j];
        if (MERGE) ss = -ss;
        o1[j] = af[j] * cc - bf[j] * ss;
        o2[j] = bf[j] * cc + af[j] * ss;
      }
      a.from_float(o1); b.from_float(o2);
    }
    a.store(dst + c);
    b.store(dst + D / 2 + c);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Dropout with a counter-based generator (Philox4x32-10): element i uses word (i % 4) of the block keyed by
// `seed` at counter (i / 4, offset).  The mask is a pure function of (seed, offset, i), so the backward pass
// regenerates it instead of storing it, and a pipelined run draws the same numbers as a sequential one.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ out, const long long* __restrict__ seed_ptr,
                               long long offset, uint32_t threshold, float scale, size_t n) {
  const unsigned long long seed = (unsigned long long)(*seed_ptr);
  const uint32_t k0 = uint32_t(seed), k1 = uint32_t(seed >> 32);
  const size_t n4 = (n + 3) / 4;
  for (size_t q = size_t(blockIdx.x) * blockDim.x + threadIdx.x; q < n4; q += size_t(gridDim.x) * blockDim.x) {
    const uint4 r = philox4x32_10(uint32_t(q), uint32_t(q >> 32), uint32_t(offset), uint32_t((unsigned long long)offset >> 32), k0, k1);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const size_t i = q * 4 + j;
      if (i < n) out[i] = T(w[j] >= threshold ? float(x[i]) * scale : 0.f);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Embedding
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                     size_t n_tok, int d, int vocab, int* status) {
  constexpr int VN = Vec<T>::N;
  const int dv = d / VN;
  const size_t total = n_tok * dv;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t t = i / dv;
    const int c = int(i % dv) * VN;
    int64_t id = ids[t];
    if (id < 0 || id >= vocab) {  // record and clamp instead of faulting
      report_status(status, JPB_ERR_BAD_ARGUMENT);
      id = 0;
    }
    Vec<T> v; v.load(table + size_t(id) * d + c);
    v.store(out + t * d + c);
  }
}

// scatter-add into an fp32 staging table (zeroed by the caller); a second pass casts to the output dtype
template <typename T>
__global__ void embedding_bwd_kernel(const T* __restrict__ dy, const int64_t* __restrict__ ids, float* __restrict__ acc,
                                     size_t n_tok, int d, int vocab) {
  constexpr int VN = Vec<T>::N;
  const int dv = d / VN;
  const size_t total = n_tok * dv;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t t = i / dv;
    const int c = int(i % dv) * VN;
    const int64_t id = ids[t];
    if (id < 0 || id >= vocab) continue;
    Vec<T> v; v.load(dy + t * d + c);
    float f[VN]; v.to_float(f);
#pragma unroll
    for (int j = 0; j < VN; ++j) atomicAdd(acc + size_t(id) * d + c + j, f[j]);
  }
}

template <typename T>
__global__ void cast_from_f32_kernel(const float* __restrict__ in, T* __restrict__ out, size_t n) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
    out[i] = from_f<T>(in[i]);
}

// ---------------------------------------------------------------------------------------------------------
// Cross entropy: one CTA per row; online (max, sum-exp) over V with 16-byte loads
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void ce_fwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ labels, float* __restrict__ loss,
                              float* __restrict__ lse_out, int rows, int V) {
  constexpr int VN = Vec<T>::N;
  __shared__ float scratch[64];
  const int nvec = (V % VN == 0) ? V / VN : 0;  // rows are only 16-byte aligned when V is a vector multiple
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* lr = logits + size_t(row) * V;
    float m = -INFINITY, s = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      Vec<T> xv; xv.load(lr + v * VN);
      float f[VN]; xv.to_float(f);
      float vm = f[0];
#pragma unroll
      for (int j = 1; j < VN; ++j) vm = fmaxf(vm, f[j]);
      if (vm > m) { s *= __expf(m - vm); m = vm; }
#pragma unroll
      for (int j = 0; j < VN; ++j) s += __expf(f[j] - m);
    }
    for (int c = nvec * VN + threadIdx.x; c < V; c += blockDim.x) {  // tail when V is not a vector multiple
      const float f = to_f(lr[c]);
      if (f > m) { s *= __expf(m - f); m = f; }
      s += __expf(f - m);
    }
    // combine (m, s) pairs across the CTA
    float wm = warp_max(m);
    s *= (m == -INFINITY) ? 0.f : __expf(m - wm);
    s = warp_sum(s);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) { scratch[warp] = wm; scratch[32 + warp] = s; }
    __syncthreads();
    float bm = lane < nwarps ? scratch[lane] : -INFINITY;
    float bs = lane < nwarps ? scratch[32 + lane] : 0.f;
    const float gm = warp_max(bm);
    bs *= (bm == -INFINITY) ? 0.f : __expf(bm - gm);
    bs = warp_sum(bs);
    if (threadIdx.x == 0) {
      const float lse = gm + logf(bs);
      const int64_t lab = labels[row];
      const float picked = (lab >= 0 && lab < V) ? to_f(lr[lab]) : 0.f;
      lse_out[row] = lse;
      loss[row] = (lab >= 0 && lab < V) ? lse - picked : 0.f;
    }
  }
}

template <typename T>
__global__ void ce_bwd_kernel(const float* __restrict__ dloss, const T* __restrict__ logits,
                              const int64_t* __restrict__ labels, const float* __restrict__ lse, T* __restrict__ dlogits,
                              int rows, int V) {
  constexpr int VN = Vec<T>::N;
  const int nvec = (V % VN == 0) ? V / VN : 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* lr = logits + size_t(row) * V;
    T* dr = dlogits + size_t(row) * V;
    const float l = lse[row], g = dloss[row];
    const int lab = int(labels[row]);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      Vec<T> xv; xv.load(lr + v * VN);
      float f[VN]; xv.to_float(f);
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        float p = __expf(f[j] - l);
        if (v * VN + j == lab) p -= 1.f;
        f[j] = p * g;
      }
      Vec<T> o; o.from_float(f); o.store(dr + v * VN);
    }
    for (int c = nvec * VN + threadIdx.x; c < V; c += blockDim.x) {
      float p = __expf(to_f(lr[c]) - l);
      if (c == lab) p -= 1.f;
      dr[c] = from_f<T>(p * g);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// AdamW: fp32 master/m/v, gradient of type G, writes new state and a low-precision copy of type O
// ---------------------------------------------------------------------------------------------------------
template <typename G, typename O>
__global__ void adamw_kernel(const float* __restrict__ p, const G* __restrict__ g, const float* __restrict__ m,
                             const float* __restrict__ v, const int64_t* __restrict__ step, float* __restrict__ p_out,
                             float* __restrict__ m_out, float* __restrict__ v_out, O* __restrict__ lp_out, size_t n, float lr,
                             float beta1, float beta2, float eps, float wd, float gscale) {
  const float t = float(*step);
  const float bc1 = 1.f - powf(beta1, t);
  const float bc2 = 1.f - powf(beta2, t);
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    const float gi = to_f(g[i]) * gscale;
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    const float upd = (mi / bc1) / (sqrtf(vi / bc2) + eps);
    const float pi = p[i] * (1.f - lr * wd) - lr * upd;
    p_out[i] = pi; m_out[i] = mi; v_out[i] = vi;
    lp_out[i] = from_f<O>(pi);
  }
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

static int norm_threads(int H, int vn, int vecs = NORM_MAX_VECS) {
  const int nvec = H / vn;
  int t = (nvec + vecs - 1) / vecs;
  t = (t + 31) / 32 * 32;
  if (t < 32) t = 32;
  return t;
}

}  // namespace jpb

using namespace jpb;
#define STREAM static_cast<cudaStream_t>(stream)
#define LAST_ERR int(cudaGetLastError())

// dtype codes used across the C ABI: 0 = fp32, 1 = bf16
template <typename F> static int dispatch_dtype(int dt, F&& f) {
  if (dt == 0) return f(float{});
  if (dt == 1) return f(__nv_bfloat16{});
  return -JPB_ERR_BAD_ARGUMENT;
}

JPB_API int jpb_norm_fwd(int layer, int dt, const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                         int rows, int H, float eps, void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec<T>::N;
    if (H % VN || H / VN > NORM_MAX_VECS * 1024) return -int(JPB_ERR_BAD_ARGUMENT);
    const int threads = norm_threads(H, VN);
    const int grid = rows < sm_count() * 8 ? rows : sm_count() * 8;
    if (layer)
      norm_fwd_kernel<T, true><<<grid, threads, 0, STREAM>>>((const T*)x, (const T*)w, (const T*)b, (T*)y, mean, rstd, rows, H, eps);
    else
      norm_fwd_kernel<T, false><<<grid, threads, 0, STREAM>>>((const T*)x, (const T*)w, nullptr, (T*)y, nullptr, rstd, rows, H, eps);
    return LAST_ERR;
  });
}

// Number of fp32 scratch elements jpb_norm_bwd needs for a given shape.
JPB_API long long jpb_norm_bwd_scratch_elems(int rows, int H) {
  const int grid = rows < sm_count() * 2 ? rows : sm_count() * 2;
  return (long long)grid * 2 * H;
}

static int norm_bwd_impl(int layer, int dt, const void* dy, const void* x, const void* w, const float* mean,
                         const float* rstd, void* dx, void* dw, void* db, float* scratch, int rows, int H, const void* add,
                         void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec<T>::N;
    if (H % VN || H / VN > NORM_BWD_VECS * 1024) return -int(JPB_ERR_BAD_ARGUMENT);
    const int threads = norm_threads(H, VN, NORM_BWD_VECS);
    const int grid = rows < sm_count() * 2 ? rows : sm_count() * 2;
    if (threads > 512) {
      if (layer)
        norm_bwd_kernel<T, true, 1024><<<grid, threads, 0, STREAM>>>((const T*)dy, (const T*)x, (const T*)w, mean, rstd, (T*)dx, scratch, rows, H, (const T*)add);
      else
        norm_bwd_kernel<T, false, 1024><<<grid, threads, 0, STREAM>>>((const T*)dy, (const T*)x, (const T*)w, nullptr, rstd, (T*)dx, scratch, rows, H, (const T*)add);
    } else if (layer) {
      norm_bwd_kernel<T, true><<<grid, threads, 0, STREAM>>>((const T*)dy, (const T*)x, (const T*)w, mean, rstd, (T*)dx, scratch, rows, H, (const T*)add);
    } else {
      norm_bwd_kernel<T, false><<<grid, threads, 0, STREAM>>>((const T*)dy, (const T*)x, (const T*)w, nullptr, rstd, (T*)dx, scratch, rows, H, (const T*)add);
    }
    reduce_partials_kernel<T><<<(H + 31) / 32, 256, 0, STREAM>>>(scratch, (T*)dw, grid, H, size_t(2) * H);
    if (layer) reduce_partials_kernel<T><<<(H + 31) / 32, 256, 0, STREAM>>>(scratch + H, (T*)db, grid, H, size_t(2) * H);
    return LAST_ERR;
  });
}

JPB_API int jpb_norm_bwd(int layer, int dt, const void* dy, const void* x, const void* w, const float* mean,
                         const float* rstd, void* dx, void* dw, void* db, float* scratch, int rows, int H, void* stream) {
  return norm_bwd_impl(layer, dt, dy, x, w, mean, rstd, dx, dw, db, scratch, rows, H, nullptr, stream);
}

// Same, with the residual-path gradient `add` (shape of dx) summed into dx in the same pass.
JPB_API int jpb_norm_bwd_add(int layer, int dt, const void* dy, const void* x, const void* w, const float* mean,
                             const float* rstd, void* dx, void* dw, void* db, float* scratch, int rows, int H,
                             const void* add, void* stream) {
  return norm_bwd_impl(layer, dt, dy, x, w, mean, rstd, dx, dw, db, scratch, rows, H, add, stream);
}

JPB_API long long jpb_colsum_scratch_elems(int rows, int cols) {
  const int parts = rows < 256 ? rows : 256;
  return (long long)parts * cols;
}

JPB_API int jpb_colsum(int dt, const void* x, void* out, float* scratch, int rows, int cols, void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec<T>::N;
    if (cols % VN) return -int(JPB_ERR_BAD_ARGUMENT);
    const int parts = rows < 256 ? rows : 256;
    const int threads = 128;
    dim3 grid((cols / VN + threads - 1) / threads, parts);
    colsum_partial_kernel<T><<<grid, threads, 0, STREAM>>>((const T*)x, scratch, rows, cols);
    reduce_partials_kernel<T><<<(cols + 31) / 32, 256, 0, STREAM>>>(scratch, (T*)out, parts, cols, size_t(cols));
    return LAST_ERR;
  });
}

static int ew_grid(size_t work, int threads) {
  size_t blocks = (work + threads - 1) / threads;
  const size_t cap = size_t(sm_count()) * 16;
  return int(blocks < cap ? (blocks ? blocks : 1) : cap);
}

// out = x * keep / (1 - p) with keep drawn from Philox keyed by *seed (an int64 on the device) at `offset`.
JPB_API int jpb_dropout(int dt, const void* x, void* out, const long long* seed, long long offset, float p, long long n,
                        void* stream) {
  if (!(p >= 0.f && p < 1.f)) return -int(JPB_ERR_BAD_ARGUMENT);
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    const double t = double(p) * 4294967296.0;
    const uint32_t threshold = t >= 4294967295.0 ? 0xFFFFFFFFu : uint32_t(t);
    dropout_kernel<T><<<ew_grid(size_t(n + 3) / 4, 256), 256, 0, STREAM>>>((const T*)x, (T*)out, seed, offset, threshold,
                                                                         1.f / (1.f - p), size_t(n));
    return LAST_ERR;
  });
}

JPB_API int jpb_gelu(int dt, int bwd, const void* x, const void* dy, void* out, long long n, void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec<T>::N;
    if (n % VN) return -int(JPB_ERR_BAD_ARGUMENT);
    const size_t nvec = n / VN;
    if (bwd) gelu_kernel<T, true><<<ew_grid(nvec, 256), 256, 0, STREAM>>>((const T*)x, (const T*)dy, (T*)out, nvec);
    else gelu_kernel<T, false><<<ew_grid(nvec, 256), 256, 0, STREAM>>>((const T*)x, nullptr, (T*)out, nvec);
    return LAST_ERR;
  });
}

JPB_API int jpb_swiglu(int dt, int bwd, const void* gu, const void* dy, void* out, long long rows, int F, void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec<T>::N;
    if (F % VN) return -int(JPB_ERR_BAD_ARGUMENT);
    const size_t work = size_t(rows) * (F / VN);
    if (bwd) swiglu_bwd_kernel<T><<<ew_grid(work, 256), 256, 0, STREAM>>>((const T*)dy, (const T*)gu, (T*)out, rows, F);
    else swiglu_fwd_kernel<T><<<ew_grid(work, 256), 256, 0, STREAM>>>((const T*)gu, (T*)out, rows, F);
    return LAST_ERR;
  });
}

JPB_API int jpb_rope(int dt, const void* x, const float* cs, const float* sn, void* out, long long bsh, int S, int H, int D,
                     int inverse, void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec<T>::N;
    if ((D / 2) % VN) return -int(JPB_ERR_BAD_ARGUMENT);
    const size_t work = size_t(bsh) * ((D / 2) / VN);
    rope_kernel<T><<<ew_grid(work, 256), 256, 0, STREAM>>>((const T*)x, cs, sn, (T*)out, bsh, S, H, D, inverse);
    return LAST_ERR;
  });
}

// merge == 0: packed -> q, k, v (RoPE on q and k unless cs is null); merge == 1: q, k, v -> packed, inverse rotation.
JPB_API int jpb_qkv_rope(int dt, int merge, void* packed, void* q, void* k, void* v, const float* cs, const float* sn,
                         long long rows, int S, int Hq, int Hkv, int D, void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec<T>::N;
    if ((D / 2) % VN) return -int(JPB_ERR_BAD_ARGUMENT);
    const size_t work = size_t(rows) * (Hq + 2 * Hkv) * ((D / 2) / VN);
    if (merge)
      qkv_rope_kernel<T, true><<<ew_grid(work, 256), 256, 0, STREAM>>>((T*)packed, (T*)q, (T*)k, (T*)v, cs, sn, rows, S, Hq, Hkv, D);
    else
      qkv_rope_kernel<T, false><<<ew_grid(work, 256), 256, 0, STREAM>>>((T*)packed, (T*)q, (T*)k, (T*)v, cs, sn, rows, S, Hq, Hkv, D);
    return LAST_ERR;
  });
}

JPB_API int jpb_embedding_fwd(int dt, const long long* ids, const void* table, void* out, long long n_tok, int d, int vocab,
                              void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec<T>::N;
    if (d % VN) return -int(JPB_ERR_BAD_ARGUMENT);
    const size_t work = size_t(n_tok) * (d / VN);
    embedding_fwd_kernel<T><<<ew_grid(work, 256), 256, 0, STREAM>>>((const int64_t*)ids, (const T*)table, (T*)out, n_tok, d, vocab,
                                                                  jpb_status_device_ptr());
    return LAST_ERR;
  });
}

// `acc` is an fp32 [vocab, d] staging buffer that this call zeroes; `out` receives the cast result
// (pass out == nullptr to keep the fp32 result in `acc` only).
JPB_API int jpb_embedding_bwd(int dt, const void* dy, const long long* ids, float* acc, void* out, long long n_tok, int d,
                              int vocab, void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec<T>::N;
    if (d % VN) return -int(JPB_ERR_BAD_ARGUMENT);
    cudaMemsetAsync(acc, 0, size_t(vocab) * d * sizeof(float), STREAM);
    const size_t work = size_t(n_tok) * (d / VN);
    embedding_bwd_kernel<T><<<ew_grid(work, 256), 256, 0, STREAM>>>((const T*)dy, (const int64_t*)ids, acc, n_tok, d, vocab);
    if (out) {
      const size_t n = size_t(vocab) * d;
      cast_from_f32_kernel<T><<<ew_grid(n, 256), 256, 0, STREAM>>>(acc, (T*)out, n);
    }
    return LAST_ERR;
  });
}

// Scatter-add of `dy` rows straight into an fp32 [vocab, d] table: with `zero_first` the table is cleared first
// (it then holds this call's gradient), without it the call adds to what is there (a gradient accumulator).
JPB_API int jpb_embedding_bwd_acc(int dt, const void* dy, const long long* ids, float* acc, long long n_tok, int d, int vocab,
                                  int zero_first, void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec<T>::N;
    if (d % VN) return -int(JPB_ERR_BAD_ARGUMENT);
    if (zero_first) cudaMemsetAsync(acc, 0, size_t(vocab) * d * sizeof(float), STREAM);
    const size_t work = size_t(n_tok) * (d / VN);
    embedding_bwd_kernel<T><<<ew_grid(work, 256), 256, 0, STREAM>>>((const T*)dy, (const int64_t*)ids, acc, n_tok, d, vocab);
    return LAST_ERR;
  });
}

JPB_API int jpb_ce_fwd(int dt, const void* logits, const long long* labels, float* loss, float* lse, int rows, int V,
                       void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    const int grid = rows < sm_count() * 4 ? rows : sm_count() * 4;
    ce_fwd_kernel<T><<<grid, 512, 0, STREAM>>>((const T*)logits, (const int64_t*)labels, loss, lse, rows, V);
    return LAST_ERR;
  });
}

JPB_API int jpb_ce_bwd(int dt, const float* dloss, const void* logits, const long long* labels, const float* lse,
                       void* dlogits, int rows, int V, void* stream) {
  return dispatch_dtype(dt, [&](auto tag) {
    using T = decltype(tag);
    const int grid = rows < sm_count() * 4 ? rows : sm_count() * 4;
    ce_bwd_kernel<T><<<grid, 512, 0, STREAM>>>(dloss, (const T*)logits, (const int64_t*)labels, lse, (T*)dlogits, rows, V);
    return LAST_ERR;
  });
}

JPB_API int jpb_adamw(int grad_dt, int out_dt, const float* p, const void* g, const float* m, const float* v,
                      const long long* step, float* p_out, float* m_out, float* v_out, void* lp_out, long long n, float lr,
                      float beta1, float beta2, float eps, float wd, float gscale, void* stream) {
  const int grid = ew_grid(size_t(n), 256);
#define ADAMW(G, O)                                                                                                      \
  adamw_kernel<G, O><<<grid, 256, 0, STREAM>>>(p, (const G*)g, m, v, (const int64_t*)step, p_out, m_out, v_out, (O*)lp_out, \
                                               size_t(n), lr, beta1, beta2, eps, wd, gscale)
  if (grad_dt == 0 && out_dt == 0) ADAMW(float, float);
  else if (grad_dt == 0 && out_dt == 1) ADAMW(float, __nv_bfloat16);
  else if (grad_dt == 1 && out_dt == 0) ADAMW(__nv_bfloat16, float);
  else if (grad_dt == 1 && out_dt == 1) ADAMW(__nv_bfloat16, __nv_bfloat16);
  else return -JPB_ERR_BAD_ARGUMENT;
#undef ADAMW
  return LAST_ERR;
}

// ---------------------------------------------------------------------------------------------------------
// RMSNorm backward without a caller-provided scratch buffer (see jaxpp_b200_noalloc.h)
// ---------------------------------------------------------------------------------------------------------
#include "jaxpp_b200_noalloc.h"

// Partial dW sums of the no-allocation entry point: [JPB_NOALLOC_MAX_PARTS][2][JPB_NOALLOC_MAX_H] floats.
static __device__ __align__(256) float g_noalloc_scratch[JPB_NOALLOC_MAX_PARTS * 2 * JPB_NOALLOC_MAX_H];
// Device address of the array above, per device; the symbol itself is only a host-side handle.
static float* g_noalloc_scratch_ptr[64] = {nullptr};

JPB_API const char* jpb_noalloc_strerror(int code) {
  switch (code) {
    case JPB_NOALLOC_OK: return "ok";
    case JPB_NOALLOC_ERR_TOO_LARGE: return "row length exceeds JPB_NOALLOC_MAX_H (8192): the built-in scratch array is too small";
    case JPB_NOALLOC_ERR_BAD_SHAPE: return "rows and H must be positive and H a multiple of 4 (float32) or 8 (bfloat16)";
    case JPB_NOALLOC_ERR_BAD_DTYPE: return "dtype must be 0 (float32) or 1 (bfloat16)";
    case JPB_NOALLOC_ERR_SETUP: return "cudaGetSymbolAddress failed for the built-in scratch array";
    default: return code > 0 ? "CUDA launch error (cudaError_t)" : "unknown error";
  }
}

JPB_API int jpb_rmsnorm_bwd_noalloc(int dtype, const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                    void* dw, int rows, int H, void* stream) {
  if (dtype != 0 && dtype != 1) return JPB_NOALLOC_ERR_BAD_DTYPE;
  const int vn = dtype == 0 ? 4 : 8;
  if (rows <= 0 || H <= 0 || H % vn != 0) return JPB_NOALLOC_ERR_BAD_SHAPE;
  if (H > JPB_NOALLOC_MAX_H) return JPB_NOALLOC_ERR_TOO_LARGE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return JPB_NOALLOC_ERR_SETUP;
  if (g_noalloc_scratch_ptr[dev] == nullptr) {
    // once per device, with that device current: turn the symbol into a device pointer
    float* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch) != cudaSuccess || ptr == nullptr)
      return JPB_NOALLOC_ERR_SETUP;
    g_noalloc_scratch_ptr[dev] = ptr;
  }
  float* scratch = g_noalloc_scratch_ptr[dev];
  const int grid = rows < JPB_NOALLOC_MAX_PARTS ? rows : JPB_NOALLOC_MAX_PARTS;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec<T>::N;
    const int threads = norm_threads(H, VN, NORM_BWD_VECS);
    // every CTA writes its whole partial row before the reduction reads it: nothing has to be cleared
    if (threads > 512)
      norm_bwd_kernel<T, false, 1024><<<grid, threads, 0, STREAM>>>((const T*)dy, (const T*)x, (const T*)w, nullptr, rstd,
                                                                    (T*)dx, scratch, rows, H);
    else
      norm_bwd_kernel<T, false><<<grid, threads, 0, STREAM>>>((const T*)dy, (const T*)x, (const T*)w, nullptr, rstd, (T*)dx,
                                                              scratch, rows, H);
    reduce_partials_kernel<T><<<(H + 31) / 32, 256, 0, STREAM>>>(scratch, (T*)dw, grid, H, size_t(2) * H);
    return LAST_ERR;
  });
}
