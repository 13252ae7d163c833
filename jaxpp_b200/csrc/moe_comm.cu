// Expert-parallel dispatch and combine fused with their all-to-all over NVLink peer memory (sm_100a).
//
// Capacity-based routing gives every (expert e, position c) slot a fixed place, so the exchange needs no
// size negotiation: rank r owns, in every peer's receive buffer, the rows that belong to "tokens of r".
//
//  dispatch  x [T, d], src_of_slot [E*C] (token row or -1), optional per-slot scale
//            -> out [E_l, n*C, d] on the rank that holds expert e (E_l = E / n experts per rank)
//            One warp per slot reads the token's row (or produces zeros for an empty slot) and stores it
//            straight into the owner's receive buffer (peer stores) -- permutation and all-to-all are the
//            same pass over the data.  Slots of local experts go directly to `out`.  When every CTA has
//            drained its stores, the last one raises this rank's flag in every peer.  The kernel then
//            waits (bounded) for each peer's flag and moves that peer's rows from the receive buffer into
//            `out`, an ordinary tensor the caller may keep for the backward pass.
//  combine   y [E_l, n*C, d], dest [T*k] (slot or E*C when dropped), optional weights [T*k]
//            -> out [T, d] = sum_j w_{t,j} * y_global[dest[t,j]],  optionally picked [T*k, d]
//            Phase 1 pushes the rows that belong to tokens of rank r into r's receive buffer (layout
//            [E, C, d]); phase 2 waits for the peers' flags and does the weighted gather-sum per token.
//
// The receive buffer is double-buffered by call parity and the flags carry an increasing epoch; every call
// receives from every peer before it ends, which keeps a peer at most one call ahead.
#include "common.cuh"

namespace jpb {

constexpr int MOE_MAX_RANKS = 8;
constexpr int MOE_THREADS = 256;

struct MoeParams {
  int n_ranks, rank, epoch;
  int n_experts, e_local, capacity, d, top_k, n_tokens;
  const __nv_bfloat16* in;       // dispatch: x [T, d]; combine: y [E_l, n*C, d]
  const int* index;              // dispatch: src_of_slot [E*C]; combine: dest [T*k]
  const float* scale;            // dispatch: per slot, combine: per (token, pick); may be null
  __nv_bfloat16* out;            // dispatch: [E_l, n*C, d]; combine: [T, d]
  __nv_bfloat16* picked;         // combine only, may be null: [T*k, d]
  __nv_bfloat16* recv_local;     // this rank's receive buffer
  __nv_bfloat16* recv_peer[MOE_MAX_RANKS];
  int* flags_local;              // [n_ranks], slot q is written by rank q
  int* flags_peer[MOE_MAX_RANKS];
  int* cta_counter;              // local, zero between calls
  int* status;
};

__device__ __forceinline__ int moe_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void moe_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 moe_ld_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 moe_scale_v4(uint4 v, float s) {
  float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), e = unpack_bf16(v.w);
  v.x = pack_bf16(a.x * s, a.y * s); v.y = pack_bf16(b.x * s, b.y * s);
  v.z = pack_bf16(c.x * s, c.y * s); v.w = pack_bf16(e.x * s, e.y * s);
  return v;
}

// All stores of this CTA are performed system-wide, then it is counted; the last CTA of the grid raises this
// rank's flag in every peer.
__device__ __forceinline__ void moe_signal_done(const MoeParams& p) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(p.cta_counter, 1) == int(gridDim.x) - 1) {
      *p.cta_counter = 0;
      __threadfence_system();
      for (int q = 0; q < p.n_ranks; ++q)
        if (q != p.rank) moe_st_release_sys(p.flags_peer[q] + p.rank, p.epoch);
    }
  }
}

// Lane 0 polls the flag of peer q (bounded); the warp learns the outcome.
__device__ __forceinline__ bool moe_wait_peer(const MoeParams& p, int q, int lane) {
  int ok = 1;
  if (lane == 0) {
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (moe_ld_acquire_sys(p.flags_local + q) < p.epoch) {
      if ((++spins & 0xff) == 0) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > wait_budget_ns()) {
          report_status(p.status, JPB_ERR_PEER_TIMEOUT);
          ok = 0;
          break;
        }
      }
    }
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__global__ void __launch_bounds__(MOE_THREADS, 4) moe_dispatch_kernel(const MoeParams p) {
  const int lane = threadIdx.x & 31;
  const int warp_g = (blockIdx.x * MOE_THREADS + threadIdx.x) >> 5;
  const int n_warps = (gridDim.x * MOE_THREADS) >> 5;
  const int nvec = p.d / 8;
  const int C = p.capacity, n = p.n_ranks;
  const long long row_stride_out = (long long)n * C;  // rows per local expert in [E_l, n*C, d]
  // ---- phase 1: every slot of every expert, remote owners first (walk owners starting after this rank) ----
  const int slots = p.n_experts * C;
  const int per_owner = p.e_local * C;
  for (int g = warp_g; g < slots; g += n_warps) {
    const int owner = (p.rank + 1 + g / per_owner) % n;
    const int in_owner = g % per_owner;
    const int el = in_owner / C, pos = in_owner % C;
    const int slot = (owner * p.e_local + el) * C + pos;
    int tok = p.index[slot];
    if (tok >= p.n_tokens) {  // an index outside the token range: record it and treat the slot as empty
      if (lane == 0) report_status(p.status, JPB_ERR_BAD_ARGUMENT);
      tok = -1;
    }
    const float s = (p.scale != nullptr && tok >= 0) ? p.scale[slot] : 1.f;
    __nv_bfloat16* base = owner == p.rank ? p.out : p.recv_peer[owner];
    __nv_bfloat16* dst = base + ((long long)el * row_stride_out + (long long)p.rank * C + pos) * p.d;
    const __nv_bfloat16* src = p.in + (long long)(tok < 0 ? 0 : tok) * p.d;
    for (int v = lane; v < nvec; v += 32) {
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (tok >= 0) {
        val = *reinterpret_cast<const uint4*>(src + v * 8);
        if (p.scale != nullptr) val = moe_scale_v4(val, s);
      }
      *reinterpret_cast<uint4*>(dst + v * 8) = val;
    }
  }
  moe_signal_done(p);
  // ---- phase 2: move what the peers sent from the receive buffer into `out` -------------------------------
  const int rows_per_peer = p.e_local * C;
  const long long total = (long long)(n - 1) * rows_per_peer;
  int verified = 0;
  for (long long g = warp_g; g < total; g += n_warps) {
    const int q = (p.rank + 1 + int(g / rows_per_peer)) % n;
    if (!(verified & (1 << q))) {
      if (!moe_wait_peer(p, q, lane)) return;
      verified |= 1 << q;
    }
    const int in_peer = int(g % rows_per_peer);
    const int el = in_peer / C, pos = in_peer % C;
    const long long row = (long long)el * row_stride_out + (long long)q * C + pos;
    const __nv_bfloat16* src = p.recv_local + row * p.d;
    __nv_bfloat16* dst = p.out + row * p.d;
    for (int v = lane; v < nvec; v += 32) *reinterpret_cast<uint4*>(dst + v * 8) = moe_ld_v4(src + v * 8);
  }
}

__global__ void __launch_bounds__(MOE_THREADS, 4) moe_combine_kernel(const MoeParams p) {
  const int lane = threadIdx.x & 31;
  const int warp_g = (blockIdx.x * MOE_THREADS + threadIdx.x) >> 5;
  const int n_warps = (gridDim.x * MOE_THREADS) >> 5;
  const int nvec = p.d / 8;
  const int C = p.capacity, n = p.n_ranks;
  const long long row_stride_in = (long long)n * C;
  // ---- phase 1: rows that belong to tokens of rank r go to r's receive buffer, laid out [E, C, d] ---------
  const int rows_per_peer = p.e_local * C;
  const long long total = (long long)(n - 1) * rows_per_peer;
  for (long long g = warp_g; g < total; g += n_warps) {
    const int r = (p.rank + 1 + int(g / rows_per_peer)) % n;
    const int in_peer = int(g % rows_per_peer);
    const int el = in_peer / C, pos = in_peer % C;
    const __nv_bfloat16* src = p.in + ((long long)el * row_stride_in + (long long)r * C + pos) * p.d;
    __nv_bfloat16* dst = p.recv_peer[r] + ((long long)(p.rank * p.e_local + el) * C + pos) * p.d;
    for (int v = lane; v < nvec; v += 32) *reinterpret_cast<uint4*>(dst + v * 8) = *reinterpret_cast<const uint4*>(src + v * 8);
  }
  moe_signal_done(p);
  // ---- phase 2: weighted gather-sum per token --------------------------------------------------------------
  for (int q = 0; q < n; ++q)
    if (q != p.rank && !moe_wait_peer(p, q, lane)) return;
  const int dump = p.n_experts * C;
  for (int t = warp_g; t < p.n_tokens; t += n_warps) {
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < p.top_k; ++j) {
        const int slot = p.index[t * p.top_k + j];
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (slot < 0 || slot > dump) {  // not a slot and not the "dropped" marker: record it, contribute nothing
          if (lane == 0 && v == lane) report_status(p.status, JPB_ERR_BAD_ARGUMENT);
        } else if (slot < dump) {
          const int e = slot / C, pos = slot % C;
          const int owner = e / p.e_local, el = e % p.e_local;
          const __nv_bfloat16* src = owner == p.rank
              ? p.in + ((long long)el * row_stride_in + (long long)p.rank * C + pos) * p.d
              : p.recv_local + (long long)slot * p.d;
          val = moe_ld_v4(src + v * 8);
          const float w = p.scale != nullptr ? p.scale[t * p.top_k + j] : 1.f;
          const float2 a = unpack_bf16(val.x), b = unpack_bf16(val.y), c = unpack_bf16(val.z), e2 = unpack_bf16(val.w);
          acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
          acc[4] += w * c.x; acc[5] += w * c.y; acc[6] += w * e2.x; acc[7] += w * e2.y;
        }
        if (p.picked != nullptr) *reinterpret_cast<uint4*>(p.picked + ((long long)t * p.top_k + j) * p.d + v * 8) = val;
      }
      uint4 o;
      o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
      o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(p.out + (long long)t * p.d + v * 8) = o;
    }
  }
}

}  // namespace jpb

// Control block: [0..7] flags written by peers, [8] local CTA counter.
struct JpbMoeDesc {
  int n_ranks, rank, epoch;
  int reserved_sms;  // SMs kept out of the grid for kernels of other streams
  void* ctrl[8];
  void* recv[8];   // receive buffer (current parity) of every rank, E*C*d bf16 each
};

JPB_API int jpb_moe_desc_bytes() { return int(sizeof(JpbMoeDesc)); }

static int moe_fill(jpb::MoeParams& p, const JpbMoeDesc* desc, int n_experts, int capacity, int d, int top_k, int n_tokens) {
  using namespace jpb;
  if (!desc || desc->n_ranks < 2 || desc->n_ranks > MOE_MAX_RANKS) return -JPB_ERR_BAD_ARGUMENT;
  if (n_experts % desc->n_ranks != 0 || d % 8 != 0 || capacity <= 0) return -JPB_ERR_BAD_ARGUMENT;
  p.n_ranks = desc->n_ranks; p.rank = desc->rank; p.epoch = desc->epoch;
  p.n_experts = n_experts; p.e_local = n_experts / desc->n_ranks; p.capacity = capacity; p.d = d;
  p.top_k = top_k; p.n_tokens = n_tokens;
  for (int q = 0; q < desc->n_ranks; ++q) {
    p.recv_peer[q] = static_cast<__nv_bfloat16*>(desc->recv[q]);
    p.flags_peer[q] = static_cast<int*>(desc->ctrl[q]);
  }
  p.recv_local = p.recv_peer[desc->rank];
  p.flags_local = p.flags_peer[desc->rank];
  p.cta_counter = p.flags_local + 8;
  p.status = jpb_status_device_ptr();
  return 0;
}

// Phase 2 of both kernels waits for flags that a peer raises only after ALL of its CTAs have finished phase 1, so
// every CTA of the grid has to be resident at once: the grid is what the occupancy calculator says fits (at most
// four CTAs per SM), less `reserved_sms` SMs left to kernels of other streams (point-to-point transfers).
template <typename K>
static int moe_grid(K kernel, int reserved_sms) {
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, jpb::MOE_THREADS, 0) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  if (per_sm > 4) per_sm = 4;
  if (reserved_sms < 0) reserved_sms = 0;
  if (reserved_sms > sms - 1) reserved_sms = sms - 1;
  return (sms - reserved_sms) * per_sm;
}

JPB_API int jpb_moe_dispatch(const void* x, const int* src_of_slot, const float* slot_scale, void* out, int n_tokens,
                             int n_experts, int capacity, int d, const JpbMoeDesc* desc, void* stream) {
  jpb::MoeParams p = {};
  const int rc = moe_fill(p, desc, n_experts, capacity, d, 0, n_tokens);
  if (rc) return rc;
  p.in = static_cast<const __nv_bfloat16*>(x); p.index = src_of_slot; p.scale = slot_scale;
  p.out = static_cast<__nv_bfloat16*>(out);
  jpb::moe_dispatch_kernel<<<moe_grid(jpb::moe_dispatch_kernel, desc->reserved_sms), jpb::MOE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return int(cudaGetLastError());
}

JPB_API int jpb_moe_combine(const void* y, const int* dest, const float* weights, void* out, void* picked, int n_tokens,
                            int top_k, int n_experts, int capacity, int d, const JpbMoeDesc* desc, void* stream) {
  jpb::MoeParams p = {};
  const int rc = moe_fill(p, desc, n_experts, capacity, d, top_k, n_tokens);
  if (rc) return rc;
  p.in = static_cast<const __nv_bfloat16*>(y); p.index = dest; p.scale = weights;
  p.out = static_cast<__nv_bfloat16*>(out); p.picked = static_cast<__nv_bfloat16*>(picked);
  jpb::moe_combine_kernel<<<moe_grid(jpb::moe_combine_kernel, desc->reserved_sms), jpb::MOE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return int(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------------
// Router: softmax over the expert logits, top-k pick, weights renormalised over the picks, and the two
// per-expert statistics of the load-balancing loss (sum of probabilities, number of picks) in one pass.
// One thread per token, at most 64 experts.
// ---------------------------------------------------------------------------------------------------------
namespace jpb {

constexpr int ROUTER_MAX_E = 64;

template <typename T>
__global__ void router_kernel(const T* __restrict__ logits, float* __restrict__ probs, long long* __restrict__ top_i,
                              float* __restrict__ weights, float* __restrict__ prob_sum, float* __restrict__ hits, int n_tok,
                              int E, int k, int* status) {
  __shared__ float s_prob[ROUTER_MAX_E];
  __shared__ float s_hits[ROUTER_MAX_E];
  for (int e = threadIdx.x; e < E; e += blockDim.x) { s_prob[e] = 0.f; s_hits[e] = 0.f; }
  __syncthreads();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < n_tok) {
    float p[ROUTER_MAX_E];
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) { p[e] = float(logits[size_t(t) * E + e]); mx = fmaxf(mx, p[e]); }
    float sum = 0.f;
    for (int e = 0; e < E; ++e) { p[e] = __expf(p[e] - mx); sum += p[e]; }
    const float inv = 1.f / sum;
    for (int e = 0; e < E; ++e) {
      p[e] *= inv;
      probs[size_t(t) * E + e] = p[e];
      atomicAdd(&s_prob[e], p[e]);
    }
    unsigned long long taken = 0ull;
    float picked = 0.f;
    int idx[8];
    float val[8];
    for (int j = 0; j < k; ++j) {
      int best = -1;
      float bv = -1.f;
      for (int e = 0; e < E; ++e)
        if (!((taken >> e) & 1ull) && p[e] > bv) { bv = p[e]; best = e; }   // ties: lowest index, like torch.topk
      if (best < 0) {
        // no comparison succeeded: the probabilities are not finite (NaN logits of a diverged step).  Take the
        // lowest expert not yet picked, so that every index stays in range, and report through the status word.
        for (int e = 0; e < E && best < 0; ++e)
          if (!((taken >> e) & 1ull)) best = e;
        bv = 0.f;
        report_status(status, JPB_ERR_BAD_ARGUMENT);
      }
      taken |= 1ull << best;
      idx[j] = best; val[j] = bv; picked += bv;
      atomicAdd(&s_hits[best], 1.f);
    }
    const float pinv = 1.f / picked;
    for (int j = 0; j < k; ++j) {
      top_i[size_t(t) * k + j] = idx[j];
      weights[size_t(t) * k + j] = val[j] * pinv;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    atomicAdd(prob_sum + e, s_prob[e]);
    atomicAdd(hits + e, s_hits[e]);
  }
}

}  // namespace jpb

// logits [n_tok, E] (fp32 dtype 0 or bf16 dtype 1) -> probs [n_tok, E] fp32, top_i [n_tok, k] int64, weights [n_tok, k]
// fp32, prob_sum [E] and hits [E] fp32 (both zeroed here).  E <= 64, k <= 8.  A token whose probabilities are not
// finite gets the lowest-numbered experts (indices stay in range) and the status word is set to JPB_ERR_BAD_ARGUMENT.
JPB_API int jpb_router(int dtype, const void* logits, float* probs, long long* top_i, float* weights, float* prob_sum,
                       float* hits, int n_tok, int E, int k, void* stream) {
  using namespace jpb;
  if (E < 1 || E > ROUTER_MAX_E || k < 1 || k > 8 || k > E) return -JPB_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaMemsetAsync(prob_sum, 0, sizeof(float) * E, s);
  cudaMemsetAsync(hits, 0, sizeof(float) * E, s);
  const int threads = 128, blocks = (n_tok + threads - 1) / threads;
  if (dtype == 0)
    router_kernel<float><<<blocks, threads, 0, s>>>(static_cast<const float*>(logits), probs, top_i, weights, prob_sum, hits, n_tok, E, k,
                                         jpb_status_device_ptr());
  else
    router_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), probs, top_i, weights,
                                                            prob_sum, hits, n_tok, E, k, jpb_status_device_ptr());
  return int(cudaGetLastError());
}
