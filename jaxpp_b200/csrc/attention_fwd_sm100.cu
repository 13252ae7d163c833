// Flash attention forward for sm_100a (causal or full, MHA/GQA, head_dim 64 or 128, bf16 in/out).
//
// One CTA handles 128 query rows of one (batch, head).  Warp 0 streams Q once and K/V blocks of 128 rows
// through a 2-stage shared-memory ring with TMA; warp 1 issues tcgen05.mma: S = Q K^T into one of two
// 128-column TMEM buffers (so S of block j+1 is computed while block j is in softmax) and O += P V into a
// third TMEM region; warps 2-9 are two softmax groups that split the 128 kv columns of a block: thread
// (row r, half g) reads its 64 columns of S from TMEM, the two halves of a row agree on the running maximum
// through shared memory (one named barrier per block), each keeps a partial sum, writes its half of P as
// bf16 into shared memory in the swizzled K-major layout the tensor core reads, rescales its half of O in
// TMEM only when some row's maximum moved, and finally normalises and stores its half of O (and the
// log-sum-exp).  The exponentials are MUFU-bound either way; two groups double the issue slots for the rest
// and halve the live registers.  All waits are bounded and report through the status word.
#include "common.cuh"

#include <cstdlib>

namespace jpb {

constexpr int ATT_BM = 128;   // query rows per CTA
constexpr int ATT_BN = 128;   // kv rows per block
// TMA warp, MMA warp and NG softmax groups of four warps; a group owns 128 / NG of the kv columns of a block (and
// D / NG of the O columns).  NG = 4 gives every scheduler four softmax warps and each thread 32 columns.
constexpr int att_threads(int ng) { return 64 + 128 * ng; }

struct AttnParams {
  int B, Sq, Sk, H, Hkv;
  int causal;
  float scale;
  __nv_bfloat16* o;   // [B, Sq, H, D]
  float* lse;         // [B, H, Sq]
  int* status;
};

template <int D>
struct AttnSmem {
  static constexpr int TILE = 128 * 64 * 2;           // one [128 rows x 64 elements] swizzled block, 16 KiB
  static constexpr int DB = D / 64;                   // 64-element blocks along head_dim
  static constexpr int Q_BYTES = DB * TILE;
  static constexpr int KV_BYTES = DB * TILE;
  static constexpr int P_BYTES = 2 * TILE;            // [128 x 128] bf16
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;       // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;  // 2 stages
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_MAX = OFF_P + P_BYTES;       // [2 block parities][up to 4 groups][128 rows] fp32 row maxima
  static constexpr int OFF_SUM = OFF_MAX + 4096;      // [up to 4 groups][128 rows] fp32 partial row sums
  static constexpr int OFF_BAR = OFF_SUM + 2048;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

// BAR_PF / BAR_PV come in pairs indexed by the parity of the kv block (two P buffers in tensor memory)
enum { BAR_Q = 0, BAR_KF = 1, BAR_VF = 3, BAR_KE = 5, BAR_VE = 7, BAR_SF = 9, BAR_SE = 11, BAR_PF = 13, BAR_PV = 15, BAR_MX = 17, BAR_N = 18 };

// PT: the probabilities go back to tensor memory (bf16, two per 32-bit column) and P V takes its A operand from
// there, instead of a round trip through shared memory (a 32 KiB store, a proxy fence and a 32 KiB operand read per
// block less on the shared-memory port, which the operand fetches of the MMAs already keep busy).  There are two such
// P buffers, used by alternate blocks: the warps write P of block j while the tensor core may still be reading P of
// block j-1, so "P handed over -> P V issued -> P V complete" (two barrier hops and the product itself, about as long
// as everything else in an iteration) leaves the loop's critical path; the warps wait for P V of the previous block
// only in the few iterations that rescale O.
template <int D, int NG, bool PT>
__global__ void __launch_bounds__(att_threads(NG), 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  using L = AttnSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + BAR_N);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.Sq + ATT_BM - 1) / ATT_BM;
  const int m_blk = num_m - 1 - blockIdx.x;  // heaviest (latest) causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int m0 = m_blk * ATT_BM;
  int n_blocks = (p.Sk + ATT_BN - 1) / ATT_BN;
  if (p.causal) {
    const int last = (m0 + ATT_BM - 1 + (p.Sk - p.Sq)) / ATT_BN + 1;
    n_blocks = last < n_blocks ? last : n_blocks;
    if (n_blocks < 1) n_blocks = 1;
  }

  if (threadIdx.x == 0) {
    mbar_init(&bar[BAR_Q], 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar[BAR_KF + s], 1);
      mbar_init(&bar[BAR_VF + s], 1);
      mbar_init(&bar[BAR_KE + s], 1);
      mbar_init(&bar[BAR_VE + s], 1);
      mbar_init(&bar[BAR_SF + s], 1);
      mbar_init(&bar[BAR_SE + s], 4 * NG);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(&bar[BAR_PF + s], 4 * NG); mbar_init(&bar[BAR_PV + s], 1); }
    mbar_init(&bar[BAR_MX], 4 * NG);   // all softmax warps meet here once per block (and once at the end)
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;
  const uint32_t tmem_p = tmem_base + 384;   // PT: P as packed bf16, two buffers of 64 columns

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------- TMA producer -------------------------------------------
      uint32_t armed = 0, armed_phase = 0;  // indexed by barrier id, for draining after an abort
      auto arm = [&](int id, uint32_t ph, uint32_t bytes) {
        mbar_expect_tx(&bar[id], bytes);
        armed |= 1u << id;
        armed_phase = (armed_phase & ~(1u << id)) | (ph << id);
      };
      arm(BAR_Q, 0, L::Q_BYTES);
#pragma unroll
      for (int d = 0; d < L::DB; ++d) tma_load_4d(smem + L::OFF_Q + d * L::TILE, &map_q, &bar[BAR_Q], d * 64, h, m0, b);
      bool ok = true;
      // K runs one block ahead of V: a K stage is free as soon as S of its block has been computed (early), a V
      // stage only after P V of its block (late).  Issued in the order K(0) K(1) V(0) K(2) V(1) ... the wait for
      // a V stage never holds back the K block that the next S needs.
      auto load_k = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait_bounded(&bar[BAR_KE + s], ph ^ 1, abort_flag, p.status)) return false;
        arm(BAR_KF + s, ph, L::KV_BYTES);
#pragma unroll
        for (int d = 0; d < L::DB; ++d)
          tma_load_4d(smem + L::OFF_K + s * L::KV_BYTES + d * L::TILE, &map_k, &bar[BAR_KF + s], d * 64, hk, j * ATT_BN, b);
        return true;
      };
      auto load_v = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait_bounded(&bar[BAR_VE + s], ph ^ 1, abort_flag, p.status)) return false;
        arm(BAR_VF + s, ph, L::KV_BYTES);
#pragma unroll
        for (int d = 0; d < L::DB; ++d)
          tma_load_4d(smem + L::OFF_V + s * L::KV_BYTES + d * L::TILE, &map_v, &bar[BAR_VF + s], d * 64, hk, j * ATT_BN, b);
        return true;
      };
      ok = load_k(0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks && !load_k(j + 1)) { ok = false; break; }
        if (!load_v(j)) { ok = false; break; }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        for (int id = 0; id < BAR_KE; ++id) {
          if (!(armed & (1u << id))) continue;
          while (!mbar_try_wait(&bar[id], (armed_phase >> id) & 1) && globaltimer_ns() - t0 < wait_budget_ns()) {
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------- MMA issuer ------------------------------------------------
      constexpr uint32_t idesc_s = make_idesc_bf16(ATT_BM, ATT_BN, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(ATT_BM, D, 0, 1);
      const uint32_t sq = smem_u32(smem + L::OFF_Q);
      const uint32_t sp = smem_u32(smem + L::OFF_P);
      bool ok = mbar_wait_bounded(&bar[BAR_Q], 0, abort_flag, p.status);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait_bounded(&bar[BAR_KF + s], ph, abort_flag, p.status)) return false;
        if (!mbar_wait_bounded(&bar[BAR_SE + s], ph ^ 1, abort_flag, p.status)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + L::OFF_K + s * L::KV_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * L::TILE + (k & 3) * 32;
          umma_bf16_ss(tmem_base + s * ATT_BN, make_smem_desc(sq + off, 16, 1024), make_smem_desc(sk + off, 16, 1024),
                       idesc_s, k != 0);
        }
        umma_commit(&bar[BAR_KE + s]);
        umma_commit(&bar[BAR_SF + s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks && !issue_s(j + 1)) { ok = false; break; }
        const int s = j & 1;
        if (!mbar_wait_bounded(&bar[BAR_PF + s], (j >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
        if (!mbar_wait_bounded(&bar[BAR_VF + s], (j >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sv = smem_u32(smem + L::OFF_V + s * L::KV_BYTES);
#pragma unroll
        for (int k = 0; k < ATT_BN / 16; ++k) {
          // A = P: K-major, two 64-wide kv blocks; B = V: MN-major, 16 kv rows per step, 64-wide d blocks
          const uint64_t db = make_smem_desc(sv + k * 2048, L::TILE, 1024);
          if constexpr (PT) {
            umma_bf16_ts(tmem_o, tmem_p + s * 64 + k * 8, db, idesc_pv, (j | k) != 0);   // 16 kv = 8 packed columns per step
          } else {
            const uint64_t da = make_smem_desc(sp + (k >> 2) * L::TILE + (k & 3) * 32, 16, 1024);
            umma_bf16_ss(tmem_o, da, db, idesc_pv, (j | k) != 0);
          }
        }
        umma_commit(&bar[BAR_VE + s]);
        umma_commit(&bar[BAR_PV + s]);
      }
    }
  } else {
    // ------------------------------------- softmax / correction / epilogue -----------------------------
    constexpr int HALF = ATT_BN / NG;           // kv columns of a block per softmax group
    constexpr int OC = D / NG;                  // O columns per softmax group
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;            // which part of the kv columns (and of the O columns)
    const int r = quarter * 32 + lane;          // row within the tile == TMEM lane
    const int qi = m0 + r;                      // query index
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    float* smax = reinterpret_cast<float*>(smem + L::OFF_MAX);
    float m_run = -INFINITY, l_run = 0.f;       // l_run: this thread's part of the row sum
    bool ok = true;
    uint8_t* sp = smem + L::OFF_P;
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int s = j & 1;
      if (!mbar_wait_bounded_warp(&bar[BAR_SF + s], (j >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
      tc_fence_after();
      float sv[HALF];
#pragma unroll
      for (int c = 0; c < HALF / 32; ++c) {
        uint32_t t[32];
        tmem_ld_32x32(tmem_base + lane_addr + s * ATT_BN + grp * HALF + c * 32, t);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[c * 32 + i] = __uint_as_float(t[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[BAR_SE + s]);  // S buffer may be overwritten by block j+2
      const int kv0 = j * ATT_BN + grp * HALF;
      const bool need_mask = (p.causal && kv0 + HALF - 1 > m0 + (p.Sk - p.Sq)) || (kv0 + HALF > p.Sk);
      if (need_mask) {
        const int limit = p.causal ? min(qi + (p.Sk - p.Sq), p.Sk - 1) : p.Sk - 1;  // last visible kv index
#pragma unroll
        for (int i = 0; i < HALF; ++i)
          if (kv0 + i > limit) sv[i] = -INFINITY;
      }
      float mx = sv[0];
#pragma unroll
      for (int i = 1; i < HALF; ++i) mx = fmaxf(mx, sv[i]);
      // the groups of a row agree on the block maximum (double-buffered by block parity, so the next
      // block's write cannot overtake a slow reader of this one)
      smax[(s * NG + grp) * ATT_BM + r] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[BAR_MX]);
      if (!mbar_wait_bounded_warp(&bar[BAR_MX], j & 1, abort_flag, p.status)) { ok = false; break; }
#pragma unroll
      for (int o = 1; o < NG; ++o) mx = fmaxf(mx, smax[(s * NG + ((grp + o) % NG)) * ATT_BM + r]);
      // Lazy rescaling: the reference maximum of a row only moves when the new maximum exceeds it by more than
      // 8 in log2 units (P then stays below 2^8, harmless in fp32 sums and bf16 P), so the read-scale-write
      // pass over O in TMEM, a chain of TMEM round trips, runs in a few blocks instead of nearly all of them.
      // All groups of a row see the same maxima and therefore take the same decision.
      const float m_cand = fmaxf(m_run, mx);
      const bool bump = (m_cand - m_run) * sl2 > 8.f;   // also true for the first finite maximum (m_run = -inf)
      const float m_new = bump ? m_cand : m_run;
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = bump ? exp2f((m_run - m_use) * sl2) : 1.f;  // 0 when m_run = -inf
      const float neg = -m_use * sl2;
      float rs = 0.f;
#pragma unroll
      for (int i = 0; i < HALF; ++i) {
        sv[i] = exp2f(fmaf(sv[i], sl2, neg));
        rs += sv[i];
      }
      l_run = l_run * alpha + rs;
      if (j > 0) {
        // P V of the previous block must be complete before O is rescaled -- and, without the second P buffer of the
        // tensor-memory path, before P is overwritten
        const bool rescale = __any_sync(0xffffffffu, bump);
        if (!PT || rescale) {
          if (!mbar_wait_bounded_warp(&bar[BAR_PV + ((j - 1) & 1)], ((j - 1) >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
        }
        if (rescale) {
#pragma unroll
          for (int c = 0; c < OC / 16; ++c) {   // this group's part of the O columns, 16 at a time
            uint32_t t[16];
            tmem_ld_32x16(tmem_o + lane_addr + grp * OC + c * 16, t);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
            tmem_st_32x16(tmem_o + lane_addr + grp * OC + c * 16, t);
          }
          tc_wait_st();
        }
      }
      if (PT && j > 1) {   // this P buffer's previous content (block j - 2) has been consumed: long since, as a rule
        if (!mbar_wait_bounded_warp(&bar[BAR_PV + s], ((j >> 1) - 1) & 1, abort_flag, p.status)) { ok = false; break; }
      }
      m_run = m_new;
      if constexpr (PT) {
        // P -> tensor memory: row r is lane r, kv columns (2c, 2c+1) share the 32-bit column c
#pragma unroll
        for (int c = 0; c < HALF / 32; ++c) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) w[i] = pack_bf16(sv[c * 32 + 2 * i], sv[c * 32 + 2 * i + 1]);
          tmem_st_32x16(tmem_p + s * 64 + lane_addr + (grp * HALF + c * 32) / 2, w);
        }
        tc_wait_st();
      } else {
        // P -> shared memory, bf16, swizzled K-major: element (r, kv) lives in block kv/64 at
        // r*128 + ((kv%64)/8 ^ (r%8))*16 + (kv%8)*2
#pragma unroll
        for (int c = 0; c < HALF / 8; ++c) {
          uint4 v;
          v.x = pack_bf16(sv[c * 8 + 0], sv[c * 8 + 1]);
          v.y = pack_bf16(sv[c * 8 + 2], sv[c * 8 + 3]);
          v.z = pack_bf16(sv[c * 8 + 4], sv[c * 8 + 5]);
          v.w = pack_bf16(sv[c * 8 + 6], sv[c * 8 + 7]);
          const int col = grp * HALF + c * 8;           // kv column of this chunk within the block
          *reinterpret_cast<uint4*>(sp + (col >> 6) * L::TILE + r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4)) = v;
        }
        fence_proxy_async();  // make the generic-proxy stores visible to the tensor core's async proxy
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[BAR_PF + s]);
    }
    if (ok && mbar_wait_bounded_warp(&bar[BAR_PV + ((n_blocks - 1) & 1)], ((n_blocks - 1) >> 1) & 1, abort_flag, p.status)) {
      tc_fence_after();
      // combine the partial row sums
      float* ssum = reinterpret_cast<float*>(smem + L::OFF_SUM);
      ssum[grp * ATT_BM + r] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[BAR_MX]);
      if (!mbar_wait_bounded_warp(&bar[BAR_MX], n_blocks & 1, abort_flag, p.status)) ok = false;
      float l_all = 0.f;
      if (ok) {
#pragma unroll
        for (int o = 0; o < NG; ++o) l_all += ssum[o * ATT_BM + r];
      }
      const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
      const bool row_ok = ok && qi < p.Sq;
      __nv_bfloat16* orow = p.o + ((size_t(b) * p.Sq + qi) * p.H + h) * D + grp * OC;
#pragma unroll
      for (int c = 0; c < OC / 16; ++c) {
        uint32_t t[16];
        tmem_ld_32x16(tmem_o + lane_addr + grp * OC + c * 16, t);
        tc_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 16; i += 8) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(t[i]) * inv, __uint_as_float(t[i + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(t[i + 2]) * inv, __uint_as_float(t[i + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(t[i + 4]) * inv, __uint_as_float(t[i + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(t[i + 6]) * inv, __uint_as_float(t[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 16 + i) = v;
          }
        }
      }
      if (row_ok && grp == 0)
        p.lse[(size_t(b) * p.H + h) * p.Sq + qi] = (l_all > 0.f) ? m_run * p.scale + logf(l_all) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// 4-D map over a [B, S, Hn, D] bf16 tensor with a box of [128 rows of S] x [64 elements of D]
static int make_bshd_map(CUtensorMap* out, const void* base, int B, int S, int Hn, int D) {
  uint64_t dims[4] = {uint64_t(D), uint64_t(Hn), uint64_t(S), uint64_t(B)};
  uint64_t strides[3] = {uint64_t(D) * 2, uint64_t(Hn) * D * 2, uint64_t(S) * Hn * D * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return jpb_make_tensor_map(out, base, 2, 4, dims, strides, box, 1);
}

// 1 (default, the faster one: 0.40 against 0.44 ms at B4 S4096 H16 D128): probabilities handed to the P V product
// through tensor memory; 0: through shared memory.  JAXPP_B200_ATTN_P_TMEM overrides the default.
static int fwd_p_tmem() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("JAXPP_B200_ATTN_P_TMEM");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v;
}

static int fwd_groups() {
  static int ng = 0;
  if (ng == 0) {
    const char* e = getenv("JAXPP_B200_ATTN_FWD_GROUPS");
    ng = (e && e[0] == '2') ? 2 : 4;
  }
  return ng;
}

template <int D, int NG, bool PT>
static int launch_attn_fwd(const void* q, const void* k, const void* v, const AttnParams& p, cudaStream_t stream) {
  using L = AttnSmem<D>;
  CUtensorMap mq, mk, mv;
  int rc = make_bshd_map(&mq, q, p.B, p.Sq, p.H, D);
  if (rc) return rc;
  rc = make_bshd_map(&mk, k, p.B, p.Sk, p.Hkv, D);
  if (rc) return rc;
  rc = make_bshd_map(&mv, v, p.B, p.Sk, p.Hkv, D);
  if (rc) return rc;
  auto kernel = attention_fwd_kernel<D, NG, PT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  dim3 grid((p.Sq + ATT_BM - 1) / ATT_BM, p.H, p.B);
  kernel<<<grid, att_threads(NG), L::TOTAL, stream>>>(mq, mk, mv, p);
  return int(cudaGetLastError());
}

}  // namespace jpb

// q: [B,Sq,H,D], k/v: [B,Sk,Hkv,D] contiguous bf16; o like q; lse: [B,H,Sq] fp32 (natural log).
JPB_API int jpb_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk, int H,
                              int Hkv, int D, int causal, float scale, void* stream) {
  using namespace jpb;
  if (H % Hkv != 0 || (D != 64 && D != 128)) return -JPB_ERR_BAD_ARGUMENT;
  AttnParams p;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.H = H; p.Hkv = Hkv; p.causal = causal; p.scale = scale;
  p.o = static_cast<__nv_bfloat16*>(o); p.lse = lse; p.status = jpb_status_device_ptr();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool pt = fwd_p_tmem() != 0;
  if (fwd_groups() == 2) {
    if (pt) return D == 128 ? launch_attn_fwd<128, 2, true>(q, k, v, p, s) : launch_attn_fwd<64, 2, true>(q, k, v, p, s);
    return D == 128 ? launch_attn_fwd<128, 2, false>(q, k, v, p, s) : launch_attn_fwd<64, 2, false>(q, k, v, p, s);
  }
  if (pt) return D == 128 ? launch_attn_fwd<128, 4, true>(q, k, v, p, s) : launch_attn_fwd<64, 4, true>(q, k, v, p, s);
  return D == 128 ? launch_attn_fwd<128, 4, false>(q, k, v, p, s) : launch_attn_fwd<64, 4, false>(q, k, v, p, s);
}
