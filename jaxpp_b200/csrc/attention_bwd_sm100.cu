// Flash attention backward for sm_100a, as two tcgen05 kernels plus a small pre-pass:
//
//   delta[b,h,q]  = sum_d dO * O                                        (attn_delta_kernel)
//   dK, dV        : one CTA per 128-row K/V block; loops over 64-row Q blocks (and, for GQA, over the
//                   query heads sharing the K/V head).  Works on transposed tiles so that each thread owns
//                   one K/V row: S^T = K Q^T, dP^T = V dO^T (TMEM), P^T and dS^T written to shared memory,
//                   dV += P^T dO and dK += dS^T Q accumulated in TMEM over the whole loop.
//   dQ            : one CTA per 128-row Q block; loops over 64-row K/V blocks: S = Q K^T, dP = dO V^T,
//                   dS to shared memory, dQ += dS K accumulated in TMEM.
//
// Recomputing S and dP in the second kernel costs two extra MMAs per tile pair but needs no atomics and no
// fp32 dQ staging buffer, and the result is deterministic.  The same shared-memory tile serves as a K-major
// operand in one MMA and as an MN-major operand in another (only the descriptor differs), so nothing is
// transposed in memory.  All waits are bounded.
#include "common.cuh"

#include <cstdlib>

namespace jpb {

// Threads of both main kernels: a TMA warp, an MMA warp and NG softmax groups of four warps.  A group owns 64 / NG of
// the 64 columns of an S tile (and D / NG of the accumulator columns in the epilogue).  NG = 4 puts four warps on
// every scheduler: each thread then holds 16 columns (half the registers) and the chain "S ready -> TMEM load ->
// exponentials -> pack -> shared memory -> hand-over", which paces the loop, is spread over twice the warps.
constexpr int bwd_threads(int ng) { return 64 + 128 * ng; }

// 32 lanes x W consecutive fp32 columns from TMEM, W = 16 or 32
template <int W>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[W]) {
  if constexpr (W == 32) tmem_ld_32x32(taddr, r);
  else tmem_ld_32x16(taddr, r);
}

struct AttnBwdParams {
  int B, Sq, Sk, H, Hkv;
  int causal;
  float scale;
  const float* lse;    // [B,H,Sq], already multiplied by log2(e)
  const float* delta;  // [B,H,Sq], already multiplied by the softmax scale
  __nv_bfloat16 *dq, *dk, *dv;
  int* status;
};

// swizzled K-major store of 8 consecutive bf16 (one 16-byte chunk `cc` of row `r`) into a [rows x 64] tile
__device__ __forceinline__ void st_swz(uint8_t* tile, int r, int cc, uint4 v) {
  *reinterpret_cast<uint4*>(tile + r * 128 + ((cc ^ (r & 7)) << 4)) = v;
}

// ---------------------------------------------------------------------------------------------------------
// Writes delta * scale and lse * log2(e): the forms the two main kernels consume, so that their inner loops are
// one fma + ex2 for P and one fma + mul for dS per element.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                  const float* __restrict__ lse, float* __restrict__ delta_s, float* __restrict__ lse2,
                                  float scale, int B, int S, int H, int D) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const long long total = (long long)B * S * H;
  if (warp >= total) return;
  const int h = warp % H;
  const long long bs = warp / H;
  const int s = int(bs % S), b = int(bs / S);
  const __nv_bfloat16* a = dO + size_t(warp) * D;
  const __nv_bfloat16* o = O + size_t(warp) * D;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 x = unpack_bf16(*reinterpret_cast<const uint32_t*>(a + i));
    const float2 y = unpack_bf16(*reinterpret_cast<const uint32_t*>(o + i));
    acc += x.x * y.x + x.y * y.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const size_t idx = (size_t(b) * H + h) * S + s;
    delta_s[idx] = acc * scale;
    lse2[idx] = lse[idx] * 1.4426950408889634f;
  }
}

// ---------------------------------------------------------------------------------------------------------
// dK / dV
// ---------------------------------------------------------------------------------------------------------
template <int D>
struct DkvSmem {
  static constexpr int DB = D / 64;
  static constexpr int KV_TILE = 128 * 128;   // [128 kv x 64 d] bf16
  static constexpr int Q_TILE = 64 * 128;     // [64 q x 64 d] bf16
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + DB * KV_TILE;
  // NS stages, each: Q (DB tiles) then dO (DB tiles).  A stage is reloaded only after the MMAs that read it have
  // completed, and a TMA load takes about as long as an iteration: with two stages the loop
  // "MMA done -> load -> S -> softmax -> MMA" spanned two iterations and set the pace; more stages hide it.
  static constexpr int NS = 4;
  static constexpr int OFF_Q = OFF_V + DB * KV_TILE;
  static constexpr int STAGE = 2 * DB * Q_TILE;
  static constexpr int OFF_P = OFF_Q + NS * STAGE;        // P^T [128 kv x 64 q] bf16, dS^T 16 KiB behind it
  static constexpr int OFF_BAR = OFF_P + 2 * 128 * 128;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

// Stages of the streamed operand (a stage is reloaded only after the MMAs that read it have completed, and a copy takes
// about as long as an iteration: three stages, tried to make room for a second pair of P^T / dS^T buffers, cost 7 %).
constexpr int DKV_NS = 4, DQ_NS = 4;
// S^T / dP^T live in two TMEM buffers (K1_SF / K1_SFREE come in pairs, indexed by the parity of the iteration): the
// tensor core computes the pair of iteration g+2 while the warps work on g and g+1, so that the round trip
// "S loaded -> next S issued -> S done" is off the loop's critical path.
enum { K1_KV = 0, K1_KVE = 1, K1_QF = 2, K1_QE = K1_QF + DKV_NS, K1_SF = K1_QE + DKV_NS, K1_SFREE = K1_SF + 2, K1_PF = K1_SFREE + 2,
       K1_PE = K1_PF + 2, K1_N = K1_PE + 2 };

// Work distribution of the persistent dK/dV kernel.  A work item is a pair of kv blocks (j, n_kvb-1-j) of one
// (batch, kv head): under a causal mask the two together see the same number of query blocks whatever j is, so
// items have equal cost and a round-robin over the CTAs is balanced; consecutive items belong to the same head
// (their Q / dO stream stays in L2).  Tile k of a CTA is half (k & 1) of its item number (k >> 1).
struct DkvTiles {
  int n_kvb, n_pairs, n_items, G, nq, causal, Sq, Sk, Hkv;
  __device__ __forceinline__ bool get(int k, int& jb, int& hk, int& b, int& i_start, int& per_head) const {
    const int item = blockIdx.x + (k >> 1) * gridDim.x;
    if (item >= n_items) return false;
    const int hb = item / n_pairs, pi = item - hb * n_pairs;
    jb = (k & 1) ? n_kvb - 1 - pi : pi;
    hk = hb % Hkv;
    b = hb / Hkv;
    i_start = 0;
    if (causal) {
      const int first_q = jb * 128 - (Sk - Sq);  // first query row that sees this kv block
      i_start = first_q > 0 ? first_q / 64 : 0;
    }
    per_head = nq > i_start ? nq - i_start : 0;
    if ((k & 1) && n_kvb - 1 - pi == pi) per_head = -1;  // odd block count: the middle block is its item's only tile
    return true;
  }
};

template <int D, int NG>
__global__ void __launch_bounds__(bwd_threads(NG), 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                     const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                     const AttnBwdParams p) {
  using L = DkvSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + K1_N);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.H / p.Hkv;
  DkvTiles tiles;
  tiles.n_kvb = (p.Sk + 127) / 128;
  tiles.n_pairs = (tiles.n_kvb + 1) / 2;
  tiles.n_items = tiles.n_pairs * p.Hkv * p.B;
  tiles.G = G; tiles.nq = (p.Sq + 63) / 64; tiles.causal = p.causal; tiles.Sq = p.Sq; tiles.Sk = p.Sk; tiles.Hkv = p.Hkv;

  if (threadIdx.x == 0) {
    mbar_init(&bar[K1_KV], 1);
    mbar_init(&bar[K1_KVE], 1);
    for (int s = 0; s < DKV_NS; ++s) { mbar_init(&bar[K1_QF + s], 1); mbar_init(&bar[K1_QE + s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bar[K1_SF + i], 1); mbar_init(&bar[K1_SFREE + i], 4 * NG); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bar[K1_PF + i], 4 * NG); mbar_init(&bar[K1_PE + i], 1); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_do); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: [S^T 64 | dP^T 64] x 2 buffers, then dV (D) and dK (D)
  const uint32_t t_dv = tmem_base + 256, t_dk = tmem_base + 256 + D;

  // Every role walks the same tiles in the same order.  `g` counts the (kv block, q block) iterations of this
  // CTA over all its tiles and `tile_i` its non-empty tiles: the barrier phases follow these two counters, so the
  // operand ring, the S / P hand-offs and the K/V buffer carry over from one tile to the next without a drain.
  if (warp == 0) {
    if (lane == 0) {
      uint32_t armed = 0, armed_phase = 0;
      auto arm = [&](int id, uint32_t ph, uint32_t bytes) {
        mbar_expect_tx(&bar[id], bytes);
        armed |= 1u << id;
        armed_phase = (armed_phase & ~(1u << id)) | (ph << id);
      };
      bool ok = true;
      uint32_t g = 0, tile_i = 0;
      int jb, hk, b, i_start, per_head;
      for (int k = 0; ok && tiles.get(k, jb, hk, b, i_start, per_head); ++k) {
        const int n_iter = per_head * G;
        if (n_iter <= 0) continue;
        // K / V of the previous tile are read by its S and dP MMAs only: free once the last of them is done
        if (tile_i > 0 && !mbar_wait_bounded(&bar[K1_KVE], (tile_i - 1) & 1, abort_flag, p.status)) { ok = false; break; }
        arm(K1_KV, tile_i & 1, 2 * L::DB * L::KV_TILE);
#pragma unroll
        for (int d = 0; d < L::DB; ++d) {
          tma_load_4d(smem + L::OFF_K + d * L::KV_TILE, &map_k, &bar[K1_KV], d * 64, hk, jb * 128, b);
          tma_load_4d(smem + L::OFF_V + d * L::KV_TILE, &map_v, &bar[K1_KV], d * 64, hk, jb * 128, b);
        }
        for (int t = 0; t < n_iter && ok; ++t, ++g) {
          const int s = g % DKV_NS;
          const uint32_t ph = (g / DKV_NS) & 1;
          const int h = hk * G + t / per_head;
          const int q0 = (i_start + t % per_head) * 64;
          if (!mbar_wait_bounded(&bar[K1_QE + s], ph ^ 1, abort_flag, p.status)) { ok = false; break; }
          arm(K1_QF + s, ph, L::STAGE);
          uint8_t* st = smem + L::OFF_Q + s * L::STAGE;
#pragma unroll
          for (int d = 0; d < L::DB; ++d) {
            tma_load_4d(st + d * L::Q_TILE, &map_q, &bar[K1_QF + s], d * 64, h, q0, b);
            tma_load_4d(st + (L::DB + d) * L::Q_TILE, &map_do, &bar[K1_QF + s], d * 64, h, q0, b);
          }
        }
        ++tile_i;
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        for (int id = 0; id < K1_QE; ++id) {
          if (id == K1_KVE || !(armed & (1u << id))) continue;
          while (!mbar_try_wait(&bar[id], (armed_phase >> id) & 1) && globaltimer_ns() - t0 < wait_budget_ns()) {
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);   // [kv x q] = K-major x K-major
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);  // [kv x d] = K-major(P^T) x MN-major(dO / Q)
      // descriptor words that do not change from one MMA to the next are computed here, once (see SmemDesc)
      const SmemDesc dk_ = make_smem_desc2(smem_u32(smem + L::OFF_K), 16, 1024);    // K, V, Q, dO, P^T, dS^T as K-major operands
      const SmemDesc dv_ = make_smem_desc2(smem_u32(smem + L::OFF_V), 16, 1024);
      const SmemDesc dq_ = make_smem_desc2(smem_u32(smem + L::OFF_Q), 16, 1024);
      const SmemDesc dp_ = make_smem_desc2(smem_u32(smem + L::OFF_P), 16, 1024);
      const SmemDesc dqm_ = make_smem_desc2(smem_u32(smem + L::OFF_Q), L::Q_TILE, 1024);   // Q / dO as MN-major operands
      constexpr uint32_t STAGE16 = L::STAGE >> 4, DO16 = (L::DB * L::Q_TILE) >> 4, DS16 = (128 * 128) >> 4;
      bool ok = true;
      auto issue_s = [&](uint32_t gg) -> bool {
        const int s = gg % DKV_NS;
        const uint32_t bf = gg & 1;
        if (!mbar_wait_bounded(&bar[K1_QF + s], (gg / DKV_NS) & 1, abort_flag, p.status)) return false;
        // the buffer's previous content (iteration gg - 2) has been read into registers
        if (gg > 1 && !mbar_wait_bounded(&bar[K1_SFREE + bf], ((gg >> 1) - 1) & 1, abort_flag, p.status)) return false;
        tc_fence_after();
        const uint32_t t_s = tmem_base + bf * 128, t_dp = t_s + 64;
        const uint32_t q_lo = dq_.lo + s * STAGE16, do_lo = q_lo + DO16;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t a_off = ((k >> 2) * L::KV_TILE + (k & 3) * 32) >> 4;
          const uint32_t b_off = ((k >> 2) * L::Q_TILE + (k & 3) * 32) >> 4;
          umma_bf16_ss2(t_s, dk_.lo + a_off, dk_.hi, q_lo + b_off, dq_.hi, idesc_s, k != 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t a_off = ((k >> 2) * L::KV_TILE + (k & 3) * 32) >> 4;
          const uint32_t b_off = ((k >> 2) * L::Q_TILE + (k & 3) * 32) >> 4;
          umma_bf16_ss2(t_dp, dv_.lo + a_off, dv_.hi, do_lo + b_off, dq_.hi, idesc_s, k != 0);
        }
        umma_commit(&bar[K1_SF + bf]);
        return true;
      };
      uint32_t g = 0, tile_i = 0;
      int jb, hk, b, i_start, per_head;
      for (int k = 0; ok && tiles.get(k, jb, hk, b, i_start, per_head); ++k) {
        const int n_iter = per_head * G;
        if (n_iter <= 0) continue;
        if (!mbar_wait_bounded(&bar[K1_KV], tile_i & 1, abort_flag, p.status)) { ok = false; break; }
        // S^T / dP^T run two iterations ahead of the products that consume P^T / dS^T
        const uint32_t g0 = g;
        int issued = 0;
        auto issue_next = [&]() -> bool {
          if (issued == n_iter) return true;
          if (!issue_s(g0 + issued)) return false;
          if (++issued == n_iter) umma_commit(&bar[K1_KVE]);  // the last S / dP of this tile: K and V may be replaced
          return true;
        };
        if (!issue_next() || !issue_next()) { ok = false; break; }
        for (int t = 0; t < n_iter && ok; ++t, ++g) {
          const int s = g % DKV_NS;
          const uint32_t pb = g & 1;
          if (!mbar_wait_bounded(&bar[K1_PF + pb], (g >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t p_lo = dp_.lo, ds_lo = p_lo + DS16;
          const uint32_t qm_lo = dqm_.lo + s * STAGE16, dom_lo = qm_lo + DO16;
          const uint32_t acc = t != 0;
#pragma unroll
          for (int kk = 0; kk < 64 / 16; ++kk)  // reduction over the 64 query rows
            umma_bf16_ss2(t_dv, p_lo + kk * 2, dp_.hi, dom_lo + kk * 128, dqm_.hi, idesc_acc, kk ? 1u : acc);
#pragma unroll
          for (int kk = 0; kk < 64 / 16; ++kk)
            umma_bf16_ss2(t_dk, ds_lo + kk * 2, dp_.hi, qm_lo + kk * 128, dqm_.hi, idesc_acc, kk ? 1u : acc);
          umma_commit(&bar[K1_QE + s]);
          umma_commit(&bar[K1_PE + pb]);
          // S^T / dP^T of iteration t + 2 (their buffer was read at the start of iteration t).  Issued after the
          // products above: with three operand stages its Q / dO may still be on their way, and a wait for them here
          // delays nothing that the warps need before iteration t + 2.
          if (!issue_next()) { ok = false; break; }
        }
        ++tile_i;
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // kv row within the block == TMEM lane
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    constexpr int CW = 64 / NG;       // query columns of an S^T tile per warp group
    constexpr int EC = D / NG;        // accumulator columns per warp group in the epilogue
    const int grp = (warp - 2) >> 2;  // which part of the 64 query columns this warp group handles
    const int cb = grp * CW;
    const int off = p.Sk - p.Sq;
    bool ok = true;
    uint32_t g = 0;
    int jb, hk, b, i_start, per_head;
    for (int k = 0; ok && tiles.get(k, jb, hk, b, i_start, per_head); ++k) {
      if (per_head < 0) continue;  // not a tile (middle block already done)
      const int n_iter = per_head * G;
      const int kv0 = jb * 128;
      const int kv = kv0 + r;
      const bool row_ok = kv < p.Sk;
      __nv_bfloat16* dk_row = p.dk + ((size_t(b) * p.Sk + kv) * p.Hkv + hk) * D;
      __nv_bfloat16* dv_row = p.dv + ((size_t(b) * p.Sk + kv) * p.Hkv + hk) * D;
      if (n_iter == 0) {
        if (row_ok) {
          for (int i = grp * EC; i < (grp + 1) * EC; i += 8) {
            *reinterpret_cast<uint4*>(dk_row + i) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(dv_row + i) = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      // Per-column statistics (lse * log2 e, delta * scale; the same addresses in every lane).  Those of iteration t + 1 are
      // requested right after the arithmetic of iteration t has consumed the current ones, into the same registers:
      // their latency then overlaps the hand-over of P^T / dS^T and the wait for the next S^T instead of standing at
      // the head of every iteration (520-610 cycles each, measured), and no extra registers are live.
      float lq[CW], dl[CW];
      auto load_stats = [&](int t) {
        const int h = hk * G + t / per_head;
        const int q0 = (i_start + t % per_head) * 64 + cb;
        const float* lse_q = p.lse + (size_t(b) * p.H + h) * p.Sq;
        const float* dl_q = p.delta + (size_t(b) * p.H + h) * p.Sq;
        if (q0 + CW - 1 < p.Sq && (p.Sq & 3) == 0) {
          const float4* l4 = reinterpret_cast<const float4*>(lse_q + q0);
          const float4* d4 = reinterpret_cast<const float4*>(dl_q + q0);
#pragma unroll
          for (int i = 0; i < CW / 4; ++i) {
            const float4 a = __ldg(l4 + i), c = __ldg(d4 + i);
            lq[4 * i] = a.x; lq[4 * i + 1] = a.y; lq[4 * i + 2] = a.z; lq[4 * i + 3] = a.w;
            dl[4 * i] = c.x; dl[4 * i + 1] = c.y; dl[4 * i + 2] = c.z; dl[4 * i + 3] = c.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < CW; ++i) {
            const bool in = q0 + i < p.Sq;
            lq[i] = in ? __ldg(lse_q + q0 + i) : 0.f;
            dl[i] = in ? __ldg(dl_q + q0 + i) : 0.f;
          }
        }
      };
      load_stats(0);
      for (int t = 0; t < n_iter && ok; ++t, ++g) {
        const int q0 = (i_start + t % per_head) * 64 + cb;
        // tile-level test (warp-uniform): is every (kv row, query column) of this warp group's 128 x CW block visible?
        const bool full = q0 + CW - 1 < p.Sq && kv0 + 127 < p.Sk && (!p.causal || kv0 + 127 <= q0 + off);
        const uint32_t bf = g & 1;
        if (!mbar_wait_bounded_warp(&bar[K1_SF + bf], (g >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        float sv[CW], dp[CW];
        {
          uint32_t a[CW], d2[CW];
          tmem_ld_cols<CW>(tmem_base + bf * 128 + lane_addr + cb, a);
          tmem_ld_cols<CW>(tmem_base + bf * 128 + 64 + lane_addr + cb, d2);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < CW; ++i) { sv[i] = __uint_as_float(a[i]); dp[i] = __uint_as_float(d2[i]); }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar[K1_SFREE + bf]);
        if (full) {
#pragma unroll
          for (int i = 0; i < CW; ++i) {
            const float pv = exp2f(fmaf(sv[i], sl2, -lq[i]));
            dp[i] = pv * fmaf(dp[i], p.scale, -dl[i]);
            sv[i] = pv;
          }
        } else {
#pragma unroll
          for (int i = 0; i < CW; ++i) {
            const int q = q0 + i;
            const bool visible = q < p.Sq && kv < p.Sk && (!p.causal || kv <= q + off);
            float pv = 0.f, ds = 0.f;
            if (visible) {
              pv = exp2f(fmaf(sv[i], sl2, -lq[i]));
              ds = pv * fmaf(dp[i], p.scale, -dl[i]);
            }
            sv[i] = pv;
            dp[i] = ds;
          }
        }
        if (t + 1 < n_iter) load_stats(t + 1);
        if (g > 0) {  // P^T / dS^T of the previous iteration (possibly of the previous tile) have been consumed
          if (!mbar_wait_bounded_warp(&bar[K1_PE + ((g - 1) & 1)], ((g - 1) >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
        }
        {
          uint8_t* tp = smem + L::OFF_P;
          uint8_t* tds = tp + 128 * 128;
#pragma unroll
          for (int c = 0; c < CW / 8; ++c) {
            uint4 v, w;
            v.x = pack_bf16(sv[c * 8 + 0], sv[c * 8 + 1]); v.y = pack_bf16(sv[c * 8 + 2], sv[c * 8 + 3]);
            v.z = pack_bf16(sv[c * 8 + 4], sv[c * 8 + 5]); v.w = pack_bf16(sv[c * 8 + 6], sv[c * 8 + 7]);
            w.x = pack_bf16(dp[c * 8 + 0], dp[c * 8 + 1]); w.y = pack_bf16(dp[c * 8 + 2], dp[c * 8 + 3]);
            w.z = pack_bf16(dp[c * 8 + 4], dp[c * 8 + 5]); w.w = pack_bf16(dp[c * 8 + 6], dp[c * 8 + 7]);
            st_swz(tp, r, grp * (CW / 8) + c, v);
            st_swz(tds, r, grp * (CW / 8) + c, w);
          }
          fence_proxy_async();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar[K1_PF + bf]);
      }
      if (!ok) break;
      // dK / dV of this tile: the accumulators are complete when the last iteration's MMAs are.  The next tile's
      // first accumulating MMA is issued only after these warps hand over its P^T / dS^T, i.e. after this read.
      if (!mbar_wait_bounded_warp(&bar[K1_PE + ((g - 1) & 1)], ((g - 1) >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = which ? t_dk : t_dv;
        __nv_bfloat16* dst = which ? dk_row : dv_row;
#pragma unroll
        for (int c = 0; c < EC / 16; ++c) {  // each warp group writes its EC of the D columns, 16 at a time
          const int col = grp * EC + c * 16;
          uint32_t a[16];
          tmem_ld_32x16(src + lane_addr + col, a);
          tc_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 16; i += 8) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(a[i]), __uint_as_float(a[i + 1]));
              v.y = pack_bf16(__uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
              v.z = pack_bf16(__uint_as_float(a[i + 4]), __uint_as_float(a[i + 5]));
              v.w = pack_bf16(__uint_as_float(a[i + 6]), __uint_as_float(a[i + 7]));
              *reinterpret_cast<uint4*>(dst + col + i) = v;
            }
          }
        }
      }
      tc_fence_before();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ---------------------------------------------------------------------------------------------------------
// dQ
// ---------------------------------------------------------------------------------------------------------
template <int D>
struct DqSmem {
  static constexpr int DB = D / 64;
  static constexpr int Q_TILE = 128 * 128;   // [128 q x 64 d]
  static constexpr int KV_TILE = 64 * 128;   // [64 kv x 64 d]
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = OFF_Q + DB * Q_TILE;
  static constexpr int OFF_KV = OFF_DO + DB * Q_TILE;   // DQ_NS stages, each: K (DB tiles) then V (DB tiles)
  static constexpr int STAGE = 2 * DB * KV_TILE;
  static constexpr int OFF_DS = OFF_KV + 4 * STAGE;     // dS [128 q x 64 kv], two buffers used by alternate iterations
  static constexpr int OFF_BAR = OFF_DS + 2 * 128 * 128;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

enum { K2_Q = 0, K2_QFREE = 1, K2_KF = 2, K2_KE = K2_KF + DQ_NS, K2_SF = K2_KE + DQ_NS, K2_SFREE = K2_SF + 2, K2_DF = K2_SFREE + 2,
       K2_DE = K2_DF + 2, K2_N = K2_DE + 2 };

// Work distribution of the persistent dQ kernel: an item is a pair of query blocks (i, num_m-1-i) of one
// (batch, head); under a causal mask the two together see the same number of kv blocks whatever i is.
struct DqTiles {
  int num_m, n_pairs, n_items, H, causal, Sq, Sk;
  __device__ __forceinline__ bool get(int k, int& m_blk, int& h, int& b, int& n_iter) const {
    const int item = blockIdx.x + (k >> 1) * gridDim.x;
    if (item >= n_items) return false;
    const int hb = item / n_pairs, pi = item - hb * n_pairs;
    m_blk = (k & 1) ? pi : num_m - 1 - pi;   // the heavier block of the pair first
    h = hb % H;
    b = hb / H;
    n_iter = (Sk + 63) / 64;
    if (causal) {
      const int last = (m_blk * 128 + 127 + (Sk - Sq)) / 64 + 1;
      n_iter = last < n_iter ? last : n_iter;
      if (n_iter < 1) n_iter = 1;
    }
    if ((k & 1) && num_m - 1 - pi == pi) n_iter = 0;  // odd block count: the middle block is its item's only tile
    return true;
  }
};

template <int D, int NG>
__global__ void __launch_bounds__(bwd_threads(NG), 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                   const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const AttnBwdParams p) {
  using L = DqSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + K2_N);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Gq = p.H / p.Hkv;
  DqTiles tiles;
  tiles.num_m = (p.Sq + 127) / 128;
  tiles.n_pairs = (tiles.num_m + 1) / 2;
  tiles.n_items = tiles.n_pairs * p.H * p.B;
  tiles.H = p.H; tiles.causal = p.causal; tiles.Sq = p.Sq; tiles.Sk = p.Sk;

  if (threadIdx.x == 0) {
    mbar_init(&bar[K2_Q], 1);
    mbar_init(&bar[K2_QFREE], 1);
    for (int s = 0; s < DQ_NS; ++s) { mbar_init(&bar[K2_KF + s], 1); mbar_init(&bar[K2_KE + s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bar[K2_SF + i], 1); mbar_init(&bar[K2_SFREE + i], 4 * NG); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bar[K2_DF + i], 4 * NG); mbar_init(&bar[K2_DE + i], 1); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_do); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_dq = tmem_base + 256;   // after the two [S 64 | dP 64] buffers

  // As in the dK/dV kernel: every role walks the same tiles; `g` counts this CTA's (q block, kv block) iterations
  // over all its tiles and `tile_i` its tiles, and the barrier phases follow those two counters.
  if (warp == 0) {
    if (lane == 0) {
      uint32_t armed = 0, armed_phase = 0;
      auto arm = [&](int id, uint32_t ph, uint32_t bytes) {
        mbar_expect_tx(&bar[id], bytes);
        armed |= 1u << id;
        armed_phase = (armed_phase & ~(1u << id)) | (ph << id);
      };
      bool ok = true;
      uint32_t g = 0, tile_i = 0;
      int m_blk, h, b, n_iter;
      for (int k = 0; ok && tiles.get(k, m_blk, h, b, n_iter); ++k) {
        if (n_iter <= 0) continue;
        const int hk = h / Gq;
        // Q / dO of the previous tile are read by its S and dP MMAs only
        if (tile_i > 0 && !mbar_wait_bounded(&bar[K2_QFREE], (tile_i - 1) & 1, abort_flag, p.status)) { ok = false; break; }
        arm(K2_Q, tile_i & 1, 2 * L::DB * L::Q_TILE);
#pragma unroll
        for (int d = 0; d < L::DB; ++d) {
          tma_load_4d(smem + L::OFF_Q + d * L::Q_TILE, &map_q, &bar[K2_Q], d * 64, h, m_blk * 128, b);
          tma_load_4d(smem + L::OFF_DO + d * L::Q_TILE, &map_do, &bar[K2_Q], d * 64, h, m_blk * 128, b);
        }
        for (int t = 0; t < n_iter && ok; ++t, ++g) {
          const int s = g % DQ_NS;
          const uint32_t ph = (g / DQ_NS) & 1;
          if (!mbar_wait_bounded(&bar[K2_KE + s], ph ^ 1, abort_flag, p.status)) { ok = false; break; }
          arm(K2_KF + s, ph, L::STAGE);
          uint8_t* st = smem + L::OFF_KV + s * L::STAGE;
#pragma unroll
          for (int d = 0; d < L::DB; ++d) {
            tma_load_4d(st + d * L::KV_TILE, &map_k, &bar[K2_KF + s], d * 64, hk, t * 64, b);
            tma_load_4d(st + (L::DB + d) * L::KV_TILE, &map_v, &bar[K2_KF + s], d * 64, hk, t * 64, b);
          }
        }
        ++tile_i;
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        for (int id = 0; id < K2_KE; ++id) {
          if (id == K2_QFREE || !(armed & (1u << id))) continue;
          while (!mbar_try_wait(&bar[id], (armed_phase >> id) & 1) && globaltimer_ns() - t0 < wait_budget_ns()) {
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);   // [q x kv]
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, D, 0, 1);   // [q x d] = K-major(dS) x MN-major(K)
      const uint32_t sq = smem_u32(smem + L::OFF_Q), sdo = smem_u32(smem + L::OFF_DO);
      const uint32_t sds0 = smem_u32(smem + L::OFF_DS);
      bool ok = true;
      auto issue_s = [&](uint32_t gg) -> bool {
        const int s = gg % DQ_NS;
        const uint32_t bf = gg & 1;
        if (!mbar_wait_bounded(&bar[K2_KF + s], (gg / DQ_NS) & 1, abort_flag, p.status)) return false;
        if (gg > 1 && !mbar_wait_bounded(&bar[K2_SFREE + bf], ((gg >> 1) - 1) & 1, abort_flag, p.status)) return false;
        tc_fence_after();
        const uint32_t t_s = tmem_base + bf * 128, t_dp = t_s + 64;
        const uint32_t sk = smem_u32(smem + L::OFF_KV + s * L::STAGE);
        const uint32_t sv = sk + L::DB * L::KV_TILE;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t a_off = (k >> 2) * L::Q_TILE + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * L::KV_TILE + (k & 3) * 32;
          umma_bf16_ss(t_s, make_smem_desc(sq + a_off, 16, 1024), make_smem_desc(sk + b_off, 16, 1024), idesc_s, k != 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t a_off = (k >> 2) * L::Q_TILE + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * L::KV_TILE + (k & 3) * 32;
          umma_bf16_ss(t_dp, make_smem_desc(sdo + a_off, 16, 1024), make_smem_desc(sv + b_off, 16, 1024), idesc_s, k != 0);
        }
        umma_commit(&bar[K2_SF + bf]);
        return true;
      };
      uint32_t g = 0, tile_i = 0;
      int m_blk, h, b, n_iter;
      for (int k = 0; ok && tiles.get(k, m_blk, h, b, n_iter); ++k) {
        if (n_iter <= 0) continue;
        if (!mbar_wait_bounded(&bar[K2_Q], tile_i & 1, abort_flag, p.status)) { ok = false; break; }
        // S / dP run two iterations ahead of the product that consumes dS
        const uint32_t g0 = g;
        int issued = 0;
        auto issue_next = [&]() -> bool {
          if (issued == n_iter) return true;
          if (!issue_s(g0 + issued)) return false;
          if (++issued == n_iter) umma_commit(&bar[K2_QFREE]);  // the last S / dP of this tile: Q and dO may be replaced
          return true;
        };
        if (!issue_next() || !issue_next()) { ok = false; break; }
        for (int t = 0; t < n_iter && ok; ++t, ++g) {
          if (!issue_next()) { ok = false; break; }   // iteration t + 2: its buffer was read at the start of iteration t
          const int s = g % DQ_NS;
          const uint32_t pb = g & 1;
          if (!mbar_wait_bounded(&bar[K2_DF + pb], (g >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sds = sds0 + pb * 128 * 128;
          const uint32_t sk = smem_u32(smem + L::OFF_KV + s * L::STAGE);
#pragma unroll
          for (int kk = 0; kk < 64 / 16; ++kk)  // reduction over the 64 kv rows
            umma_bf16_ss(t_dq, make_smem_desc(sds + kk * 32, 16, 1024), make_smem_desc(sk + kk * 2048, L::KV_TILE, 1024),
                         idesc_dq, (t | kk) != 0);
          umma_commit(&bar[K2_KE + s]);
          umma_commit(&bar[K2_DE + pb]);
        }
        ++tile_i;
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    const int off = p.Sk - p.Sq;
    constexpr int CW = 64 / NG;       // kv columns of an S tile per warp group
    constexpr int EC = D / NG;        // dQ columns per warp group in the epilogue
    const int grp = (warp - 2) >> 2;  // which part of the 64 kv columns this warp group handles
    const int cb = grp * CW;
    bool ok = true;
    uint32_t g = 0;
    int m_blk, h, b, n_iter;
    for (int k = 0; ok && tiles.get(k, m_blk, h, b, n_iter); ++k) {
      if (n_iter <= 0) continue;
      const int m0 = m_blk * 128;
      const int qi = m0 + r;
      const bool row_ok = qi < p.Sq;
      const float lse_r = row_ok ? p.lse[(size_t(b) * p.H + h) * p.Sq + qi] : 0.f;
      const float dl_r = row_ok ? p.delta[(size_t(b) * p.H + h) * p.Sq + qi] : 0.f;
      for (int t = 0; t < n_iter && ok; ++t, ++g) {
        const uint32_t bf = g & 1;
        if (!mbar_wait_bounded_warp(&bar[K2_SF + bf], (g >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        float sv[CW], dp[CW];
        {
          uint32_t a[CW], d2[CW];
          tmem_ld_cols<CW>(tmem_base + bf * 128 + lane_addr + cb, a);
          tmem_ld_cols<CW>(tmem_base + bf * 128 + 64 + lane_addr + cb, d2);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < CW; ++i) { sv[i] = __uint_as_float(a[i]); dp[i] = __uint_as_float(d2[i]); }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar[K2_SFREE + bf]);
        // warp-uniform: every (query row, kv column) of this warp group's 128 x CW block visible?
        const int kv_first = t * 64 + cb;
        const bool full = m0 + 127 < p.Sq && kv_first + CW - 1 < p.Sk && (!p.causal || kv_first + CW - 1 <= m0 + off);
        if (full) {
#pragma unroll
          for (int i = 0; i < CW; ++i) {
            const float pv = exp2f(fmaf(sv[i], sl2, -lse_r));
            dp[i] = pv * fmaf(dp[i], p.scale, -dl_r);
          }
        } else {
#pragma unroll
          for (int i = 0; i < CW; ++i) {
            const int kv = kv_first + i;
            const bool visible = row_ok && kv < p.Sk && (!p.causal || kv <= qi + off);
            float ds = 0.f;
            if (visible) {
              const float pv = exp2f(fmaf(sv[i], sl2, -lse_r));
              ds = pv * fmaf(dp[i], p.scale, -dl_r);
            }
            dp[i] = ds;
          }
        }
        if (g > 1) {  // this buffer's previous content (iteration g - 2, possibly of the previous tile) has been consumed
          if (!mbar_wait_bounded_warp(&bar[K2_DE + bf], ((g >> 1) - 1) & 1, abort_flag, p.status)) { ok = false; break; }
        }
        {
          uint8_t* tds = smem + L::OFF_DS + bf * 128 * 128;
#pragma unroll
          for (int c = 0; c < CW / 8; ++c) {
            uint4 w;
            w.x = pack_bf16(dp[c * 8 + 0], dp[c * 8 + 1]); w.y = pack_bf16(dp[c * 8 + 2], dp[c * 8 + 3]);
            w.z = pack_bf16(dp[c * 8 + 4], dp[c * 8 + 5]); w.w = pack_bf16(dp[c * 8 + 6], dp[c * 8 + 7]);
            st_swz(tds, r, grp * (CW / 8) + c, w);
          }
          fence_proxy_async();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar[K2_DF + bf]);
      }
      if (!ok) break;
      // dQ of this tile; the next tile's first accumulating MMA needs a dS hand-over from these warps, which comes
      // after this read of the accumulator
      if (!mbar_wait_bounded_warp(&bar[K2_DE + ((g - 1) & 1)], ((g - 1) >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
      tc_fence_after();
      __nv_bfloat16* dst = p.dq + ((size_t(b) * p.Sq + qi) * p.H + h) * D;
#pragma unroll
      for (int c = 0; c < EC / 16; ++c) {
        const int col = grp * EC + c * 16;
        uint32_t a[16];
        tmem_ld_32x16(t_dq + lane_addr + col, a);
        tc_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 16; i += 8) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(a[i]), __uint_as_float(a[i + 1]));
            v.y = pack_bf16(__uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
            v.z = pack_bf16(__uint_as_float(a[i + 4]), __uint_as_float(a[i + 5]));
            v.w = pack_bf16(__uint_as_float(a[i + 6]), __uint_as_float(a[i + 7]));
            *reinterpret_cast<uint4*>(dst + col + i) = v;
          }
        }
      }
      tc_fence_before();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// 4-D map over [B, S, Hn, D] bf16 with a box of [rows of S] x [64 elements of D]
static int make_map_rows(CUtensorMap* out, const void* base, int B, int S, int Hn, int D, int rows) {
  uint64_t dims[4] = {uint64_t(D), uint64_t(Hn), uint64_t(S), uint64_t(B)};
  uint64_t strides[3] = {uint64_t(D) * 2, uint64_t(Hn) * D * 2, uint64_t(S) * Hn * D * 2};
  uint32_t box[4] = {64, 1, uint32_t(rows), 1};
  return jpb_make_tensor_map(out, base, 2, 4, dims, strides, box, 1);
}

// Softmax groups per CTA of the two backward kernels: 2 (default; 3-5 % faster than 4 in every measurement: the loop is
// paced by the operand fetches of the MMAs, not by the warps) or 4.  JAXPP_B200_ATTN_BWD_GROUPS overrides the default.
static int bwd_groups() {
  static int ng = 0;
  if (ng == 0) {
    const char* e = getenv("JAXPP_B200_ATTN_BWD_GROUPS");
    ng = (e && e[0] == '4') ? 4 : 2;
  }
  return ng;
}

template <int D, int NG>
static int launch_bwd(const void* dO, const void* q, const void* k, const void* v, const AttnBwdParams& p, cudaStream_t stream) {
  CUtensorMap mq64, mdo64, mk128, mv128, mq128, mdo128, mk64, mv64;
  int rc = 0;
  rc |= make_map_rows(&mq64, q, p.B, p.Sq, p.H, D, 64);
  rc |= make_map_rows(&mdo64, dO, p.B, p.Sq, p.H, D, 64);
  rc |= make_map_rows(&mk128, k, p.B, p.Sk, p.Hkv, D, 128);
  rc |= make_map_rows(&mv128, v, p.B, p.Sk, p.Hkv, D, 128);
  rc |= make_map_rows(&mq128, q, p.B, p.Sq, p.H, D, 128);
  rc |= make_map_rows(&mdo128, dO, p.B, p.Sq, p.H, D, 128);
  rc |= make_map_rows(&mk64, k, p.B, p.Sk, p.Hkv, D, 64);
  rc |= make_map_rows(&mv64, v, p.B, p.Sk, p.Hkv, D, 64);
  if (rc) return rc;
  auto k1 = attn_bwd_dkdv_kernel<D, NG>;
  auto k2 = attn_bwd_dq_kernel<D, NG>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvSmem<D>::TOTAL) != cudaSuccess) return -3;
    if (cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem<D>::TOTAL) != cudaSuccess) return -3;
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int n_kvb = (p.Sk + 127) / 128;
  const int items = ((n_kvb + 1) / 2) * p.Hkv * p.B;  // pairs of kv blocks, see DkvTiles
  const int g1 = items < sms ? items : sms;
  k1<<<g1, bwd_threads(NG), DkvSmem<D>::TOTAL, stream>>>(mq64, mdo64, mk128, mv128, p);
  const int num_m = (p.Sq + 127) / 128;
  const int items2 = ((num_m + 1) / 2) * p.H * p.B;  // pairs of query blocks, see DqTiles
  const int g2 = items2 < sms ? items2 : sms;
  k2<<<g2, bwd_threads(NG), DqSmem<D>::TOTAL, stream>>>(mq128, mdo128, mk64, mv64, p);
  return int(cudaGetLastError());
}

}  // namespace jpb

// Scratch needed by jpb_attention_bwd: two fp32 vectors [B,H,Sq] (delta * scale, lse * log2 e).
JPB_API long long jpb_attention_bwd_scratch_bytes(int B, int Sq, int Sk, int H, int Hkv, int D) {
  (void)Sk; (void)Hkv; (void)D;
  return (long long)B * H * Sq * 4 * 2;
}

// All tensors contiguous bf16: dO/q/o/dq [B,Sq,H,D], k/v/dk/dv [B,Sk,Hkv,D]; lse [B,H,Sq] fp32.
// `scratch` must hold jpb_attention_bwd_scratch_bytes(); `reserved` is unused (pass NULL).
JPB_API int jpb_attention_bwd(const void* dO, const void* q, const void* k, const void* v, const void* o, const float* lse,
                              void* dq, void* dk, void* dv, void* scratch, void* reserved, int B, int Sq, int Sk, int H,
                              int Hkv, int D, int causal, float scale, void* stream) {
  using namespace jpb;
  (void)reserved;
  if (H % Hkv != 0 || (D != 64 && D != 128)) return -JPB_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* delta = static_cast<float*>(scratch);
  float* lse2 = delta + (size_t)B * H * Sq;
  const long long rows = (long long)B * Sq * H;
  const int threads = 256;
  const long long blocks = (rows * 32 + threads - 1) / threads;
  attn_delta_kernel<<<(unsigned)blocks, threads, 0, s>>>(static_cast<const __nv_bfloat16*>(dO),
                                                         static_cast<const __nv_bfloat16*>(o), lse, delta, lse2, scale,
                                                         B, Sq, H, D);
  AttnBwdParams p;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.H = H; p.Hkv = Hkv; p.causal = causal; p.scale = scale;
  p.lse = lse2; p.delta = delta;
  p.dq = static_cast<__nv_bfloat16*>(dq); p.dk = static_cast<__nv_bfloat16*>(dk); p.dv = static_cast<__nv_bfloat16*>(dv);
  p.status = jpb_status_device_ptr();
  if (bwd_groups() == 2) return D == 128 ? launch_bwd<128, 2>(dO, q, k, v, p, s) : launch_bwd<64, 2>(dO, q, k, v, p, s);
  return D == 128 ? launch_bwd<128, 4>(dO, q, k, v, p, s) : launch_bwd<64, 4>(dO, q, k, v, p, s);
}
