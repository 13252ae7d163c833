// All-reduce over NVLink peer memory in one kernel: reduce-scatter (each rank sums its slice of every peer's
// buffer with direct peer loads, applies a scale, accumulates in fp32) followed by an all-gather of the reduced
// slices, for gradient synchronisation across data-/tensor-parallel replicas (sum + scale + cast fused).
//
// Layout: every rank has a symmetric buffer X of `n` elements (its contribution, staged before the launch).
//   phase 1  rank r reduces elements [r*S, (r+1)*S) over all ranks' X and writes the result back into its own X
//            (other ranks read only *their* slices of this X, so the in-place write does not race);
//   barrier  the last CTA to finish phase 1 raises this rank's "slice ready" flag in every peer;
//   phase 2  every rank copies the reduced slices out of the owners' X into its output tensor.
// NVSwitch gives every pair full bandwidth, so the one-shot direct pattern (no ring) is used.  All waits on peer
// flags are bounded; flags carry an increasing epoch; X is double-buffered by call parity by the caller.
//
// The two halves also run alone, for optimizer state sharded over the data-parallel ranks:
//   reduce-scatter (mode 1)  phase 1 only; `out` is this rank's reduced slice [n / n_ranks] (gradient shard);
//   all-gather     (mode 2)  every rank staged its slice at the start of X; phase 2 only, `out` is [n] (the
//                            updated low-precision parameters, gathered from the owners of the shards).
// A rank leaves call e+1 only after every peer has started call e+1, i.e. finished call e, so the buffer of call
// e is no longer read by anyone when call e+2 stages into it: parity double-buffering covers all three modes.
#include "common.cuh"

namespace jpb {

constexpr int AR_MAX_RANKS = 8;

struct AllReduceParams {
  int n_ranks, rank, epoch;
  int mode;                   // 0 all-reduce, 1 reduce-scatter, 2 all-gather
  long long n;                // elements
  float scale;
  void* x[AR_MAX_RANKS];      // symmetric buffers (x[rank] is local)
  int* ready_peer[AR_MAX_RANKS];   // [n_ranks] ints in each rank's control block: ready_peer[q][r] = epoch when r staged X
  int* slice_peer[AR_MAX_RANKS];   // [n_ranks] ints: slice_peer[q][r] = epoch when r finished reducing its slice
  int* ready_local;
  int* slice_local;
  unsigned int* cta_counter;  // local, monotonically increasing
  unsigned int counter_target;
  void* out;                  // [n] result
  int* status;
};

__device__ __forceinline__ int ar_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ar_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ar_ld_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// One thread of the CTA waits (bounded) for all peers' flags; the CTA learns the outcome through shared memory.
__device__ __forceinline__ bool ar_wait_all(const int* flags, int n_ranks, int rank, int epoch, int* status, int* smem_ok) {
  if (threadIdx.x == 0) {
    int ok = 1;
    uint64_t t0 = 0;   // the clock is read every 256 polls only (a read costs about as much as a small all-reduce step)
    for (int q = 0; q < n_ranks && ok; ++q) {
      if (q == rank) continue;
      uint32_t spins = 0;
      while (ar_ld_acquire_sys(flags + q) < epoch) {
        if ((++spins & 0xff) == 0) {
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > wait_budget_ns()) {
            report_status(status, JPB_ERR_PEER_TIMEOUT);
            ok = 0;
            break;
          }
        }
      }
    }
    *smem_ok = ok;
  }
  __syncthreads();
  return *smem_ok != 0;
}

// Copy `count` 16-byte vectors, four loads in flight per thread (peer loads have microseconds of latency: the
// bandwidth of a link is reached only with several MB outstanding per GPU).
__device__ __forceinline__ void ar_copy_vec(uint8_t* dst, const uint8_t* src, long long count) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; v + 3 * stride < count; v += 4 * stride) {
    const uint4 a = ar_ld_v4(src + v * 16), b = ar_ld_v4(src + (v + stride) * 16);
    const uint4 c = ar_ld_v4(src + (v + 2 * stride) * 16), d = ar_ld_v4(src + (v + 3 * stride) * 16);
    *reinterpret_cast<uint4*>(dst + v * 16) = a;
    *reinterpret_cast<uint4*>(dst + (v + stride) * 16) = b;
    *reinterpret_cast<uint4*>(dst + (v + 2 * stride) * 16) = c;
    *reinterpret_cast<uint4*>(dst + (v + 3 * stride) * 16) = d;
  }
  for (; v < count; v += stride) *reinterpret_cast<uint4*>(dst + v * 16) = ar_ld_v4(src + v * 16);
}

template <typename T>
__device__ __forceinline__ void ar_accumulate(float* acc, const uint4& in) {
  if constexpr (sizeof(T) == 4) {
    acc[0] += __uint_as_float(in.x); acc[1] += __uint_as_float(in.y);
    acc[2] += __uint_as_float(in.z); acc[3] += __uint_as_float(in.w);
  } else {
    const float2 a = unpack_bf16(in.x), b = unpack_bf16(in.y), c = unpack_bf16(in.z), d = unpack_bf16(in.w);
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
  }
}

template <typename T>
__device__ __forceinline__ uint4 ar_pack(const float* acc, float scale) {
  uint4 o;
  if constexpr (sizeof(T) == 4) {
    o.x = __float_as_uint(acc[0] * scale); o.y = __float_as_uint(acc[1] * scale);
    o.z = __float_as_uint(acc[2] * scale); o.w = __float_as_uint(acc[3] * scale);
  } else {
    o.x = pack_bf16(acc[0] * scale, acc[1] * scale); o.y = pack_bf16(acc[2] * scale, acc[3] * scale);
    o.z = pack_bf16(acc[4] * scale, acc[5] * scale); o.w = pack_bf16(acc[6] * scale, acc[7] * scale);
  }
  return o;
}

template <typename T>
__global__ void __launch_bounds__(512) allreduce_kernel(const AllReduceParams p) {
  __shared__ int ok_flag;
  constexpr int VN = 16 / sizeof(T);
  const long long nvec = p.n / VN;                       // n is a multiple of VN * n_ranks (checked on the host)
  const long long slice = nvec / p.n_ranks;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (int q = 0; q < p.n_ranks; ++q)
      if (q != p.rank) ar_st_release_sys(p.ready_peer[q] + p.rank, p.epoch);  // my X is staged (stream order)
  }
  if (!ar_wait_all(p.ready_local, p.n_ranks, p.rank, p.epoch, p.status, &ok_flag)) return;

  if (p.mode == 2) {
    // ---- all-gather only: every rank's slice sits at the start of its X ------------------------------------
    for (int s = 0; s < p.n_ranks; ++s) {
      const int q = (p.rank + s) % p.n_ranks;
      ar_copy_vec(static_cast<uint8_t*>(p.out) + slice * q * 16, static_cast<const uint8_t*>(p.x[q]), slice);
    }
    return;
  }
  // ---- phase 1: reduce my slice -----------------------------------------------------------------------
  const long long base = slice * p.rank;
  const long long obase = p.mode == 1 ? 0 : base;   // reduce-scatter: `out` holds the slice only
  {
    constexpr int U = 4;   // vectors per thread and pass: U loads in flight per peer
    const long long stride = (long long)gridDim.x * blockDim.x;
    uint8_t* xo = static_cast<uint8_t*>(p.x[p.rank]) + base * 16;
    uint8_t* oo = static_cast<uint8_t*>(p.out) + obase * 16;
    for (long long v0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; v0 < slice; v0 += U * stride) {
      float acc[U][VN];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < VN; ++j) acc[u][j] = 0.f;
      for (int q = 0; q < p.n_ranks; ++q) {
        const uint8_t* xq = static_cast<const uint8_t*>(p.x[q]) + base * 16;
        uint4 in[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long v = v0 + u * stride;
          in[u] = v < slice ? ar_ld_v4(xq + v * 16) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) ar_accumulate<T>(acc[u], in[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + u * stride;
        if (v < slice) {
          const uint4 o = ar_pack<T>(acc[u], p.scale);
          if (p.mode == 0) *reinterpret_cast<uint4*>(xo + v * 16) = o;
          *reinterpret_cast<uint4*>(oo + v * 16) = o;
        }
      }
    }
  }
  if (p.mode == 1) return;
  // ---- barrier: the last CTA of this rank publishes the slice to the peers ---------------------------------
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(p.cta_counter, 1u) + 1u;
    if (done == p.counter_target) {
      for (int q = 0; q < p.n_ranks; ++q)
        if (q != p.rank) ar_st_release_sys(p.slice_peer[q] + p.rank, p.epoch);
    }
  }
  if (!ar_wait_all(p.slice_local, p.n_ranks, p.rank, p.epoch, p.status, &ok_flag)) return;

  // ---- phase 2: gather the other ranks' reduced slices --------------------------------------------------------
  for (int s = 1; s < p.n_ranks; ++s) {
    const int q = (p.rank + s) % p.n_ranks;
    ar_copy_vec(static_cast<uint8_t*>(p.out) + slice * q * 16, static_cast<const uint8_t*>(p.x[q]) + slice * q * 16, slice);
  }
}

}  // namespace jpb

struct JpbAllReduceDesc {
  int n_ranks, rank, epoch, dtype;   // dtype: 0 fp32, 1 bf16
  long long n;
  float scale;
  unsigned int counter_target;       // cumulative CTA count expected after this call
  void* x[8];
  void* ctrl[8];                     // control blocks: ints [0..7] ready, [8..15] slice, [16] CTA counter
  void* out;
  int grid;
  int mode;                          // 0 all-reduce, 1 reduce-scatter (out = slice), 2 all-gather (x = slice)
};

JPB_API int jpb_allreduce_desc_bytes() { return int(sizeof(JpbAllReduceDesc)); }

// Grid of an all-reduce over `n_elems` elements.  The kernel's CTAs wait for one another (the last one to finish
// phase 1 raises the flags the others poll), so all of them must be resident at once: at most one 512-thread CTA
// per SM, checked against the occupancy calculator, less `reserved_sms` SMs left to kernels of other streams.
JPB_API int jpb_allreduce_grid2(long long n_elems, int elem_bytes, int reserved_sms) {
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, jpb::allreduce_kernel<float>, 512, 0) != cudaSuccess || per_sm < 1)
    return 1;   // cannot show that more than one CTA fits: a grid of one needs no co-residency
  if (reserved_sms < 0) reserved_sms = 0;
  if (reserved_sms > sms - 1) reserved_sms = sms - 1;
  const long long cap = sms - reserved_sms;
  const long long nvec = n_elems * elem_bytes / 16;
  long long blocks = (nvec + 511) / 512;
  if (blocks < 1) blocks = 1;
  return int(blocks < cap ? blocks : cap);
}
JPB_API int jpb_allreduce_grid(long long n_elems, int elem_bytes) { return jpb_allreduce_grid2(n_elems, elem_bytes, 0); }

// In-place semantics on the staged symmetric buffers; `out` receives scale * sum over ranks.
// n must be a multiple of (16 / elem_bytes) * n_ranks.
JPB_API int jpb_allreduce(const JpbAllReduceDesc* d, void* stream) {
  using namespace jpb;
  if (!d || d->n_ranks < 2 || d->n_ranks > AR_MAX_RANKS) return -JPB_ERR_BAD_ARGUMENT;
  const int vn = d->dtype == 0 ? 4 : 8;
  if (d->n <= 0 || d->n % (vn * d->n_ranks) != 0) return -JPB_ERR_BAD_ARGUMENT;
  if (d->mode < 0 || d->mode > 2) return -JPB_ERR_BAD_ARGUMENT;
  AllReduceParams p;
  p.n_ranks = d->n_ranks; p.rank = d->rank; p.epoch = d->epoch; p.n = d->n; p.scale = d->scale; p.mode = d->mode;
  for (int q = 0; q < d->n_ranks; ++q) {
    p.x[q] = d->x[q];
    int* c = static_cast<int*>(d->ctrl[q]);
    p.ready_peer[q] = c;
    p.slice_peer[q] = c + 8;
  }
  int* mine = static_cast<int*>(d->ctrl[d->rank]);
  p.ready_local = mine;
  p.slice_local = mine + 8;
  p.cta_counter = reinterpret_cast<unsigned int*>(mine + 16);
  p.counter_target = d->counter_target;
  p.out = d->out;
  p.status = jpb_status_device_ptr();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (d->dtype == 0) allreduce_kernel<float><<<d->grid, 512, 0, s>>>(p);
  else allreduce_kernel<__nv_bfloat16><<<d->grid, 512, 0, s>>>(p);
  return int(cudaGetLastError());
}
