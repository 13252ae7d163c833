// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a).
//
// One persistent kernel per op; the tcgen05 main loop is the one of gemm_sm100.cu (TMA ring -> tcgen05.mma
// -> double-buffered TMEM accumulators -> epilogue warps) plus four "comm" warps per CTA.
//
//  all-gather -> GEMM   Every rank owns a symmetric buffer G[n_ranks][rows_per_rank, width].  The comm warps
//                       of rank r PUSH r's shard straight from the tensor it lives in into slot r of every
//                       peer's G (coalesced 16-byte peer stores, posted writes, each byte crosses the link
//                       once, no staging copy), in 16 KiB pieces spread over all comm warps of the grid; the
//                       warp that completes a chunk raises the chunk's flag in the receiver's memory.  The
//                       TMA producer reads the tiles (or k-blocks) of the own shard directly from the shard
//                       (its own tensor map) and runs them first; it waits on the chunk flag before it
//                       touches a chunk a peer pushes.  The gather can be along the rows of A (forward /
//                       dgrad) or along the reduction dimension (wgrad).  Optionally the comm warps also
//                       assemble the complete gathered operand in an ordinary local tensor (own shard +
//                       received chunks) while the tensor cores work, for a later local GEMM.
//  GEMM -> reduce-scatter
//                       Output row block p belongs to rank p.  The epilogue of a tile of a peer's block
//                       stores the bf16 partial tile straight into the owner's receive buffer (128-byte row
//                       segments through a shared-memory transpose) and then raises a per-tile flag in the
//                       owner's memory; the epilogue of an own tile waits for the peers' flags, adds the
//                       received partials in fp32 and writes the final tile.  Peer and own tiles alternate in
//                       groups of 16 row tiles (peers first), which spreads the link traffic over the kernel.
//  reduction gather with an fp32 output (wgrad) runs one pass over the tiles per rank slot, the own slot
//                       first, accumulating into D, so that no tile waits mid-k-loop for data in flight.
//
// Buffers are double-buffered by call parity, flags carry a monotonically increasing epoch and are never
// reset.  No multicast load is used anywhere.  Every wait (mbarrier, chunk flag, peer flag) is bounded.
#include "common.cuh"

namespace jpb {

constexpr int CBM = 128, CBN = 256, CBK = 64, CUMMA_K = 16;
constexpr int CSTAGES = 4;
constexpr int CA_BYTES = CBM * CBK * 2;
constexpr int CB_BYTES = CBN * CBK * 2;
constexpr int CSTAGE_BYTES = CA_BYTES + CB_BYTES;
constexpr int COMM_WARPS = 4;
constexpr int COMM_THREADS = 32 * (6 + COMM_WARPS);  // TMA, MMA, 4 epilogue warps, comm warps
constexpr int EPI_STAGE_BYTES = 4 * 32 * 128;        // per epilogue warp: 32 rows x 64 bf16, swizzled
constexpr int CSMEM_BYTES = CSTAGES * CSTAGE_BYTES + EPI_STAGE_BYTES + 1024 + 256;
constexpr int MAX_RANKS = 8;
constexpr int PIECE_BYTES = 16384;

enum GatherMode : int { GATHER_NONE = 0, GATHER_ROWS = 1, GATHER_RED = 2 };

struct CommGemmParams {
  int M, N, K;
  int ldd, out_fp32, accumulate, bias_fp32;
  const void* bias;
  void* D;
  int* status;
  int tiles_m, tiles_n;
  int a_blocked, b_blocked;          // MN-major operand through a 3-D map {64, K, MN/64}: one copy per stage
  // --- collective ---
  int n_ranks, rank;
  int epoch;                         // > 0, increases with every call on this workspace
  // all-gather
  int gather;                        // GatherMode
  int gathered_is_b;                 // GATHER_RED: which operand is the gathered one
  int phases;                        // GATHER_RED with fp32 output: one pass over all tiles per rank slot (see kernel)
  int chunks_per_rank;               // m-tiles (GATHER_ROWS) or k-blocks (GATHER_RED) per rank slot
  int rows_per_slot;                 // rows of G per rank slot
  int pieces;                        // pieces per chunk
  long long chunk_bytes;             // contiguous bytes of one chunk inside G
  long long piece_bytes;
  const uint8_t* own_src;            // this rank's shard [rows_per_slot, width], contiguous
  uint8_t* gather_out;               // optional: complete gathered operand, assembled locally
  uint8_t* g_local;                  // this rank's G
  uint8_t* g_peer[MAX_RANKS];        // every rank's G as mapped here (g_peer[rank] == g_local)
  int* chunk_flags;                  // local, [n_ranks * chunks_per_rank], slot q is written by rank q
  int* chunk_flags_peer[MAX_RANKS];  // the same array in every peer's memory
  int* piece_count;                  // local scratch, [n_ranks * chunks_per_rank], zero between calls
  // reduce-scatter
  int scatter;                       // 0/1
  __nv_bfloat16* r_local;            // receive buffer [n_ranks][rows_per_rank, N] (slot = source rank)
  __nv_bfloat16* r_peer[MAX_RANKS];
  int* tile_flags_local;             // [n_ranks][tiles_m_per_rank * tiles_n]
  int* tile_flags_peer[MAX_RANKS];
  int rows_per_rank;                 // M / n_ranks for scatter
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Spin until *flag >= want (flags only grow), at most the wait budget (jpb_set_wait_budget_ns).  The poll is a relaxed load and one
// acquire fence follows the successful one: an acquire load at system scope per poll measured about 2 us each
// on this hardware, which added up to tens of microseconds per CTA in the reduction-gather.
__device__ __forceinline__ bool flag_wait_bounded(const int* flag, int want, bool sys, volatile int* abort_flag, int* status,
                                                  int code) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (true) {
    const int v = *reinterpret_cast<const volatile int*>(flag);
    if (v >= want) {
      if (sys) asm volatile("fence.acq_rel.sys;" ::: "memory");
      else asm volatile("fence.acq_rel.gpu;" ::: "memory");
      return true;
    }
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > wait_budget_ns()) {
        *abort_flag = 1;
        report_status(status, code);
        return false;
      }
    }
  }
}

// Four consecutive flags (16-byte aligned) with one load per poll; an acquire fence orders what follows.
__device__ __forceinline__ bool flag_wait4_bounded(const int* flags, int want, volatile int* abort_flag, int* status, int code) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (true) {
    int4 v;
    asm volatile("ld.volatile.global.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(flags) : "memory");
    if (v.x >= want && v.y >= want && v.z >= want && v.w >= want) {
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      return true;
    }
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > wait_budget_ns()) {
        *abort_flag = 1;
        report_status(status, code);
        return false;
      }
    }
  }
}

// Wait until `count` consecutive flags are all >= want, with relaxed loads (several in flight) and a single
// acquire fence at the end: a pass of the reduction-gather needs a whole slot, and one fence is much cheaper
// than an acquire per chunk.
__device__ __forceinline__ bool flags_wait_all_bounded(const int* flags, int count, int want, volatile int* abort_flag,
                                                       int* status, int code) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  int done = 0;  // flags [0, done) have been seen
  while (done < count) {
    bool all = true;
    int i = done;
    for (; i + 4 <= count && all; i += 4) {
      int a, b, c, d;
      if (((reinterpret_cast<uintptr_t>(flags + i)) & 15) == 0) {
        asm volatile("ld.volatile.global.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(flags + i) : "memory");
      } else {
        a = *reinterpret_cast<const volatile int*>(flags + i);     b = *reinterpret_cast<const volatile int*>(flags + i + 1);
        c = *reinterpret_cast<const volatile int*>(flags + i + 2); d = *reinterpret_cast<const volatile int*>(flags + i + 3);
      }
      all = a >= want && b >= want && c >= want && d >= want;
      if (all) done = i + 4;
    }
    for (; i < count && all; ++i) {
      all = *reinterpret_cast<const volatile int*>(flags + i) >= want;
      if (all) done = i + 1;
    }
    if (done >= count) break;
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > wait_budget_ns()) {
        *abort_flag = 1;
        report_status(status, code);
        return false;
      }
    }
  }
  asm volatile("fence.acq_rel.sys;" ::: "memory");
  return true;
}

// Tile order.  Plain: groups of 16 row tiles walked column by column (L2-friendly).  Row gather: the own row
// block first, then the peers' blocks in the order their chunks arrive.  Scatter: the row blocks of all ranks
// are interleaved in groups of 16 row tiles -- group g of the next rank's block, of the one after, ..., of the
// own block last, then group g+1 -- so that the NVLink traffic is spread over the kernel instead of being
// crammed into its first (n-1)/n, while an own tile still runs a group (more than a wave of the grid) after
// the peers computed its partials.  (Interleaving column by column put both in the same wave and every own
// tile waited for the link: measured 30 % slower on the K = 2048 projection.)
struct TileOrder {
  int tiles_m, tiles_n, n_ranks, rank, tm_per_rank, mode;  // mode: 0 plain, 1 own-first, 2 scatter (interleaved)
  __device__ __forceinline__ void get(int idx, int& m_blk, int& n_blk) const {
    if (mode == 2) {
      const int per_group = 16 * tiles_n * n_ranks;
      const int group = idx / per_group, first_m = group * 16;
      const int gm = (tm_per_rank - first_m) < 16 ? (tm_per_rank - first_m) : 16;
      const int ing = idx - group * per_group;            // [n_ranks][tiles_n][gm]
      const int per_blk = tiles_n * gm;
      const int blk = ing / per_blk;
      const int rem = ing - blk * per_blk;
      n_blk = rem / gm;
      const int l = rem - n_blk * gm;
      const int slot = (rank + 1 + blk) % n_ranks;        // blk == n_ranks - 1 is the own block
      m_blk = slot * tm_per_rank + first_m + l;
      return;
    }
    const int rows_here = mode == 0 ? tiles_m : tm_per_rank;
    const int per_block = rows_here * tiles_n;
    const int blk = idx / per_block, in = idx % per_block;
    const int per_group = 16 * tiles_n;
    const int group = in / per_group, first_m = group * 16;
    const int gm = (rows_here - first_m) < 16 ? (rows_here - first_m) : 16;
    const int ing = in - group * per_group;
    const int lm = first_m + ing % gm;
    n_blk = ing / gm;
    if (mode == 0) {
      m_blk = lm;
      return;
    }
    const int slot = (rank + blk) % n_ranks;
    m_blk = slot * tm_per_rank + lm;
  }
};

__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// One warp copies `len` bytes (a multiple of 16, both pointers 16-byte aligned) with 16 loads in flight per lane.
__device__ __forceinline__ void copy_piece(uint8_t* dst, const uint8_t* src, long long len, int lane) {
  const long long nvec = len / 16;
  long long v = lane;
  for (; v + 15 * 32 < nvec; v += 16 * 32) {
    uint4 r[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) r[u] = ld_volatile_v4(src + (v + u * 32) * 16);
#pragma unroll
    for (int u = 0; u < 16; ++u) *reinterpret_cast<uint4*>(dst + (v + u * 32) * 16) = r[u];
  }
  for (; v < nvec; v += 32) *reinterpret_cast<uint4*>(dst + v * 16) = ld_volatile_v4(src + v * 16);
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(COMM_THREADS, 1)
comm_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_own, const CommGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + CSTAGES * CSTAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + CSTAGES * CSTAGE_BYTES + EPI_STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + CSTAGES;
  uint64_t* acc_full = bars + 2 * CSTAGES;
  uint64_t* acc_empty = bars + 2 * CSTAGES + 2;
  uint64_t* epi_bar = bars + 2 * CSTAGES + 4;  // the four epilogue warps meet here before a tile flag is raised
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * CSTAGES + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = (p.K + CBK - 1) / CBK;
  TileOrder order;
  order.tiles_m = p.tiles_m; order.tiles_n = p.tiles_n; order.n_ranks = p.n_ranks; order.rank = p.rank;
  order.tm_per_rank = p.tiles_m / p.n_ranks;
  order.mode = p.scatter ? 2 : (p.gather == GATHER_ROWS ? 1 : 0);
  const int k_rot = p.gather == GATHER_RED ? p.rank * p.chunks_per_rank : 0;
  // Reduction-gather with an fp32 output runs in `phases` passes over this CTA's tiles: pass 0 multiplies the own
  // rank's slice of the reduction dimension, pass q the slice pushed by rank (rank + q) % n, each adding into D
  // through the accumulate epilogue.  No tile ever waits in the middle of its k loop for data still in flight:
  // by the time pass q starts, the tensor cores have spent a whole pass on data that was already here.  The
  // same CTA (and the same thread) owns a tile in every pass, so the read-modify-write of D needs no fence.
  const int phases = p.phases;
  const int kb_per_pass = phases > 1 ? p.chunks_per_rank : k_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < CSTAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    mbar_init(epi_bar, 4);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (p.gather != GATHER_NONE) tma_prefetch_desc(&map_own);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------ TMA producer ------------------------------------------
    if (lane == 0) {
      uint32_t it = 0, armed = 0, armed_phase = 0;
      bool ok = true;
      // Chunk flags only grow, so a chunk seen once stays valid: in reduction-gather mode every tile walks
      // the same chunks in the same order and only the first tile of this CTA polls.
      int red_verified = 0;
      auto chunk_ready = [&](int chunk) -> bool {
        if (!flag_wait_bounded(p.chunk_flags + chunk, p.epoch, true, abort_flag, p.status, JPB_ERR_PEER_TIMEOUT)) return false;
        fence_proxy_async_global();
        return true;
      };
      // own ranges, so that the k loop below needs no division
      const int own_row0 = p.rank * p.rows_per_slot;
      const int own_lo = p.rank * p.chunks_per_rank, own_hi = own_lo + p.chunks_per_rank;
      const bool rows_mode = p.gather == GATHER_ROWS, red_mode = p.gather == GATHER_RED;
      const bool gathered_a = red_mode && !p.gathered_is_b, gathered_b = red_mode && p.gathered_is_b;
      for (int pass = 0; pass < phases && ok; ++pass) {
      const int pass_slot = (p.rank + pass) % p.n_ranks;
      if (phases > 1) {
        // a new slice: all of its chunks must have landed (they had a whole pass of tensor-core time to do so)
        if (pass > 0) {
          if (!flags_wait_all_bounded(p.chunk_flags + pass_slot * p.chunks_per_rank, p.chunks_per_rank, p.epoch, abort_flag,
                                      p.status, JPB_ERR_PEER_TIMEOUT)) { ok = false; break; }
          fence_proxy_async_global();
        }
        red_verified = kb_per_pass;
      }
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        order.get(tile, m_blk, n_blk);
        const int m0 = m_blk * CBM, n0 = n_blk * CBN;
        const bool own_rows = rows_mode && m_blk >= own_lo && m_blk < own_hi;
        if (rows_mode && !own_rows && !chunk_ready(m_blk)) { ok = false; break; }
        int kbe = phases > 1 ? pass_slot * p.chunks_per_rank : k_rot;
        for (int kb = 0; kb < kb_per_pass; ++kb, ++it, kbe = (kbe + 1 == k_blocks ? 0 : kbe + 1)) {
          const bool own_k = red_mode && kbe >= own_lo && kbe < own_hi;
          if (red_mode && !own_k && kb >= red_verified) {
            // four chunks per poll where the flags are aligned and none of the four is an own chunk
            if ((kbe & 3) == 0 && kbe + 3 < k_blocks && !(kbe < own_lo && kbe + 3 >= own_lo)) {
              if (!flag_wait4_bounded(p.chunk_flags + kbe, p.epoch, abort_flag, p.status, JPB_ERR_PEER_TIMEOUT)) { ok = false; break; }
              fence_proxy_async_global();
              red_verified = kb + 4;
            } else {
              if (!chunk_ready(kbe)) { ok = false; break; }
              red_verified = kb + 1;
            }
          }
          const int s = it % CSTAGES;
          const uint32_t ph = (it / CSTAGES) & 1;
          if (!mbar_wait_bounded(&empty[s], ph ^ 1, abort_flag, p.status)) { ok = false; break; }
          uint8_t* sa = smem + s * CSTAGE_BYTES;
          uint8_t* sb = sa + CA_BYTES;
          mbar_expect_tx(&full[s], CSTAGE_BYTES);
          armed |= 1u << s;
          armed_phase = (armed_phase & ~(1u << s)) | (ph << s);
          const int k0 = kbe * CBK;
          if (!A_MN) {
            if (own_rows) tma_load_2d(sa, &map_own, &full[s], k0, m0 - own_row0);
            else tma_load_2d(sa, &map_a, &full[s], k0, m0);
          } else {
            const bool a_own = own_k && gathered_a;
            const CUtensorMap* ma = a_own ? &map_own : &map_a;
            const int ka = a_own ? k0 - own_row0 : k0;
            if (p.a_blocked) {
              tma_load_3d(sa, ma, &full[s], 0, ka, m0 >> 6);
            } else {
#pragma unroll
              for (int j = 0; j < CBM / 64; ++j) tma_load_2d(sa + j * 8192, ma, &full[s], m0 + j * 64, ka);
            }
          }
          if (!B_MN) {
            tma_load_2d(sb, &map_b, &full[s], k0, n0);
          } else {
            const bool b_own = own_k && gathered_b;
            const CUtensorMap* mb = b_own ? &map_own : &map_b;
            const int kbk = b_own ? k0 - own_row0 : k0;
            if (p.b_blocked) {
              tma_load_3d(sb, mb, &full[s], 0, kbk, n0 >> 6);
            } else {
#pragma unroll
              for (int j = 0; j < CBN / 64; ++j) tma_load_2d(sb + j * 8192, mb, &full[s], n0 + j * 64, kbk);
            }
          }
        }
      }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        for (int s = 0; s < CSTAGES; ++s) {
          if (!(armed & (1u << s))) continue;
          while (!mbar_try_wait(&full[s], (armed_phase >> s) & 1) && globaltimer_ns() - t0 < wait_budget_ns()) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------ MMA issuer --------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(CBM, CBN, A_MN, B_MN);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      for (int pass = 0; pass < phases && ok; ++pass)
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_i) {
        const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait_bounded(&acc_empty[acc], acc_ph ^ 1, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * CBN;
        for (int kb = 0; kb < kb_per_pass; ++kb, ++it) {
          const int s = it % CSTAGES;
          if (!mbar_wait_bounded(&full[s], (it / CSTAGES) & 1, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * CSTAGE_BYTES), sb = sa + CA_BYTES;
#pragma unroll
          for (int k = 0; k < CBK / CUMMA_K; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16_ss(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full[acc]);
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------ comm warps: push the own shard to every peer ------------
    if (p.gather != GATHER_NONE) {
      const int n_comm = gridDim.x * COMM_WARPS;
      const int wid = (warp - 6) * gridDim.x + blockIdx.x;
      const int per_chunk = (p.n_ranks - 1) * p.pieces;
      const long long total = (long long)p.chunks_per_rank * per_chunk;
      for (long long g = wid; g < total; g += n_comm) {
        const int c = int(g / per_chunk), rem = int(g % per_chunk);
        const int pi = rem / p.pieces, piece = rem % p.pieces;
        const int q = (p.rank + p.n_ranks - 1 - pi) % p.n_ranks;  // the peer that consumes this shard first goes first
        const long long off = (long long)c * p.chunk_bytes + (long long)piece * p.piece_bytes;
        const long long left = p.chunk_bytes - (long long)piece * p.piece_bytes;
        const long long len = left < p.piece_bytes ? left : p.piece_bytes;
        copy_piece(p.g_peer[q] + (long long)p.rank * p.chunks_per_rank * p.chunk_bytes + off, p.own_src + off, len, lane);
        __threadfence_system();  // the stores of every lane are performed at the peer before the count below
        __syncwarp();
        if (lane == 0) {
          int* cnt = p.piece_count + pi * p.chunks_per_rank + c;
          if (atomicAdd(cnt, 1) == p.pieces - 1) {
            *cnt = 0;  // ready for the next call; nobody else touches it before
            __threadfence_system();
            st_release_sys(p.chunk_flags_peer[q] + p.rank * p.chunks_per_rank + c, p.epoch);
          }
        }
      }
      if (p.gather_out != nullptr) {
        // assemble the complete gathered operand locally: own shard first, then the chunks peers pushed
        const long long own_total = (long long)p.chunks_per_rank * p.pieces;
        const long long all_total = own_total * p.n_ranks;
        bool ok = true;
        for (long long g = wid; g < all_total && ok; g += n_comm) {
          const int blk = int(g / own_total);           // 0: own slot, then in consumption order
          const int slot = (p.rank + blk) % p.n_ranks;
          const long long in = g % own_total;
          const int c = int(in / p.pieces), piece = int(in % p.pieces);
          const long long off = (long long)c * p.chunk_bytes + (long long)piece * p.piece_bytes;
          const long long left = p.chunk_bytes - (long long)piece * p.piece_bytes;
          const long long len = left < p.piece_bytes ? left : p.piece_bytes;
          const long long slot_off = (long long)slot * p.chunks_per_rank * p.chunk_bytes;
          const uint8_t* src = p.own_src + off;
          if (blk != 0) {
            int w = 1;
            if (lane == 0)
              w = flag_wait_bounded(p.chunk_flags + slot * p.chunks_per_rank + c, p.epoch, true, abort_flag, p.status,
                                    JPB_ERR_PEER_TIMEOUT);
            w = __shfl_sync(0xffffffffu, w, 0);
            if (!w) { ok = false; break; }
            src = p.g_local + slot_off + off;
          }
          copy_piece(p.gather_out + slot_off + off, src, len, lane);
        }
      }
    }
  } else {
    // ------------------------------------------ epilogue (warps 2..5) -----------------------------------
    const int quarter = warp & 3;
    const int tm_per_rank = order.tm_per_rank;
    const int tiles_per_rank = tm_per_rank * p.tiles_n;
    uint32_t tile_i = 0, epi_uses = 0;
    bool ok = true;
    for (int pass = 0; pass < phases && ok; ++pass)
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_i) {
      int m_blk, n_blk;
      order.get(tile, m_blk, n_blk);
      const int m0 = m_blk * CBM, n0 = n_blk * CBN;
      const bool accumulate = p.accumulate || pass > 0;
      const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
      if (!mbar_wait_bounded_warp(&acc_full[acc], acc_ph, abort_flag, p.status)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const int owner = p.scatter ? m_blk / tm_per_rank : p.rank;
      const int lm = p.scatter ? m_blk % tm_per_rank : m_blk;
      const int local_row = p.scatter ? lm * CBM + quarter * 32 + lane : row;
      const bool remote = p.scatter && owner != p.rank;
      if (p.scatter && !remote) {
        // own block: the peers' partials for this tile must have landed
        int w = 1;
        if (lane == 0) {  // one lane polls and fences; the shuffle below orders the other lanes after it
          for (int q = 0; q < p.n_ranks && w; ++q) {
            if (q == p.rank) continue;
            w = flag_wait_bounded(p.tile_flags_local + q * tiles_per_rank + lm * p.tiles_n + n_blk, p.epoch, true, abort_flag,
                                  p.status, JPB_ERR_PEER_TIMEOUT);
          }
        }
        w = __shfl_sync(0xffffffffu, w, 0);
        if (!w) { ok = false; break; }
      }
      if (remote) {
        // Partial tile for a peer: transpose through shared memory so that every store instruction of the
        // warp writes four complete 128-byte row segments into the owner's receive buffer.
        uint8_t* stg = epi_stage + (warp - 2) * (32 * 128);
        __nv_bfloat16* dst_rows = p.r_peer[owner] + (size_t(p.rank) * p.rows_per_rank + lm * CBM + quarter * 32) * p.N;
#pragma unroll 1
        for (int c2 = 0; c2 < CBN / 64; ++c2) {
          const int col0 = n0 + c2 * 64;
          if (col0 >= p.N) break;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + acc * CBN + c2 * 64 + half * 32, r);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
              o.y = pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              o.z = pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              o.w = pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              *reinterpret_cast<uint4*>(stg + lane * 128 + (((half * 4 + j) ^ (lane & 7)) * 16)) = o;
            }
          }
          __syncwarp();
          const int vec = lane & 7;
          const int col = col0 + vec * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = i * 4 + (lane >> 3);
            const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((vec ^ (rr & 7)) * 16));
            if (col < p.N) *reinterpret_cast<uint4*>(dst_rows + size_t(rr) * p.N + col) = o;
          }
          __syncwarp();
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < CBN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + acc * CBN + c * 32, r);
        tc_wait_ld();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (!row_ok) continue;
        const int ncols = (p.N - col0) < 32 ? (p.N - col0) : 32;  // N is a multiple of 8
        if (p.scatter) {
          for (int q = 0; q < p.n_ranks; ++q) {
            if (q == p.rank) continue;
            const __nv_bfloat16* s = p.r_local + (size_t(q) * p.rows_per_rank + local_row) * p.N + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (j < ncols) {
                const uint4 in = ld_volatile_v4(s + j);
                const float2 a = unpack_bf16(in.x), b2 = unpack_bf16(in.y), c2 = unpack_bf16(in.z), d2 = unpack_bf16(in.w);
                v[j] += a.x; v[j + 1] += a.y; v[j + 2] += b2.x; v[j + 3] += b2.y;
                v[j + 4] += c2.x; v[j + 5] += c2.y; v[j + 6] += d2.x; v[j + 7] += d2.y;
              }
            }
          }
        }
        if (p.bias && pass == 0) {
          if (p.bias_fp32) {
            const float* b = static_cast<const float*>(p.bias) + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) if (j < ncols) v[j] += __ldg(b + j);
          } else {
            const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(p.bias) + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) if (j < ncols) v[j] += __bfloat162float(b[j]);
          }
        }
        if (p.out_fp32) {
          float* d = static_cast<float*>(p.D) + size_t(local_row) * p.ldd + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (j < ncols) {
              float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              if (accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(d + j);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(d + j) = o;
            }
          }
        } else {
          __nv_bfloat16* d = static_cast<__nv_bfloat16*>(p.D) + size_t(local_row) * p.ldd + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (j < ncols) {
              uint4 o;
              o.x = pack_bf16(v[j], v[j + 1]); o.y = pack_bf16(v[j + 2], v[j + 3]);
              o.z = pack_bf16(v[j + 4], v[j + 5]); o.w = pack_bf16(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(d + j) = o;
            }
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (remote) {
        // all four warps' peer stores must be visible before the owner sees the tile flag
        __threadfence_system();
        __syncwarp();
        if (lane == 0) mbar_arrive(epi_bar);
        if (!mbar_wait_bounded_warp(epi_bar, epi_uses & 1, abort_flag, p.status)) { ok = false; break; }
        ++epi_uses;
        if (warp == 2 && lane == 0)
          st_release_sys(p.tile_flags_peer[owner] + p.rank * tiles_per_rank + lm * p.tiles_n + n_blk, p.epoch);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// 3-D bf16 map over an MN-major operand stored as [k_rows, mn contiguous], mn a multiple of 64 (see gemm_sm100.cu)
static int comm_map_mn_blocked(CUtensorMap* out, const void* base, uint64_t mn, uint64_t k_rows, uint64_t ld_elems, uint32_t blocks) {
  uint64_t dims[3] = {64, k_rows, mn / 64};
  uint64_t strides[2] = {ld_elems * 2, 128};
  uint32_t box[3] = {64, 64, blocks};
  return jpb_make_tensor_map(out, base, 2, 3, dims, strides, box, 1);
}

// 2-D bf16 tensor map (row-major, `cols` contiguous)
static int comm_map_2d(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t ld_elems, uint32_t box_cols,
                       uint32_t box_rows) {
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {ld_elems * 2};
  uint32_t box[2] = {box_cols, box_rows};
  return jpb_make_tensor_map(out, base, 2, 2, dims, strides, box, 1);
}

template <bool A_MN, bool B_MN>
static int comm_launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const CommGemmParams& p,
                       int max_ctas, cudaStream_t stream) {
  auto kernel = comm_gemm_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CSMEM_BYTES) != cudaSuccess) return -3;
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // At most one CTA per SM, so the whole grid is co-resident: the comm warps of every CTA push while the
  // producers of the peer wait for what they push.
  // A cap below the SM count keeps SMs free for kernels this one does not know about (point-to-point
  // transfers of a pipeline on other streams), which must be able to run while CTAs here wait for a peer.
  const int tiles = p.tiles_m * p.tiles_n;
  int grid = tiles < sms ? tiles : sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  kernel<<<grid, COMM_THREADS, CSMEM_BYTES, stream>>>(ma, mb, mo, p);
  return int(cudaGetLastError());
}

}  // namespace jpb

// Layout of the per-rank control block (ints) inside the symmetric workspace.
#define JPB_MAX_CHUNKS 4096
#define JPB_CTRL_CHUNK_FLAGS 16                        /* [JPB_MAX_CHUNKS] written by peers */
#define JPB_CTRL_PIECE_COUNT (16 + JPB_MAX_CHUNKS)     /* [JPB_MAX_CHUNKS] local scratch, zero between calls */
#define JPB_CTRL_TILE_FLAGS (16 + 2 * JPB_MAX_CHUNKS)  /* [8 * JPB_MAX_TILES_PER_RANK] written by peers */
#define JPB_MAX_TILES_PER_RANK 8192
#define JPB_CTRL_INTS (JPB_CTRL_TILE_FLAGS + 8 * JPB_MAX_TILES_PER_RANK)

struct JpbCommDesc {
  int n_ranks, rank, epoch;
  int gather;            // 0 none, 1 rows of A, 2 reduction dimension
  int gathered_is_b;     // which operand is read from G (its pointer argument is ignored)
  int scatter;
  int max_ctas;          // > 0: cap on the grid (leaves SMs free for kernels of other streams), 0: one CTA per SM
  void* ctrl[8];         // control block of every rank as mapped in this process
  void* g[8];            // gather buffer (current parity) of every rank
  void* r[8];            // receive buffer (current parity) of every rank
};

JPB_API long long jpb_comm_ctrl_bytes() { return (long long)JPB_CTRL_INTS * 4; }
JPB_API int jpb_comm_desc_bytes() { return int(sizeof(JpbCommDesc)); }  // lets a binding check its struct layout

// D = A * B^T with a fused all-gather of one operand and/or reduce-scatter of the output (see file header).
// For gather != 0 the gathered operand's pointer argument (A or B) is this rank's SHARD [rows / n_ranks, width]
// (bf16, contiguous); the complete operand G is [n_ranks * rows_per_rank, width]:
//   gather == 1: A = G is [M, K] K-major;  gather == 2: the gathered operand is MN-major, G is [K, M] or [K, N].
// gather_out (optional, gather != 0): receives the complete gathered operand.
// For scatter != 0, D is this rank's [M / n_ranks, N] block.
JPB_API int jpb_comm_gemm(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int lda, int ldb,
                          int ldd, int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int bias_fp32,
                          const JpbCommDesc* desc, void* gather_out, void* stream) {
  using namespace jpb;
  if (!desc || desc->n_ranks < 2 || desc->n_ranks > MAX_RANKS) return -JPB_ERR_BAD_ARGUMENT;
  const int n = desc->n_ranks;
  if (M % (CBM * n) != 0 && (desc->scatter || desc->gather == GATHER_ROWS)) return -JPB_ERR_BAD_ARGUMENT;
  if (desc->gather == GATHER_RED && K % (CBK * n) != 0) return -JPB_ERR_BAD_ARGUMENT;
  if (N % 8 != 0 || (accumulate && !out_fp32)) return -JPB_ERR_BAD_ARGUMENT;
  CommGemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.out_fp32 = out_fp32; p.accumulate = accumulate; p.bias_fp32 = bias_fp32;
  p.bias = bias; p.D = D; p.status = jpb_status_device_ptr();
  p.tiles_m = (M + CBM - 1) / CBM;
  p.tiles_n = (N + CBN - 1) / CBN;
  p.n_ranks = n; p.rank = desc->rank; p.epoch = desc->epoch;
  p.phases = 1;
  p.gather = desc->gather; p.scatter = desc->scatter;
  int* my_ctrl = static_cast<int*>(desc->ctrl[desc->rank]);
  p.chunk_flags = my_ctrl + JPB_CTRL_CHUNK_FLAGS;
  p.piece_count = my_ctrl + JPB_CTRL_PIECE_COUNT;
  p.gathered_is_b = desc->gathered_is_b;
  p.tile_flags_local = my_ctrl + JPB_CTRL_TILE_FLAGS;
  for (int q = 0; q < n; ++q) {
    int* c = static_cast<int*>(desc->ctrl[q]);
    p.chunk_flags_peer[q] = c + JPB_CTRL_CHUNK_FLAGS;
    p.tile_flags_peer[q] = c + JPB_CTRL_TILE_FLAGS;
    p.g_peer[q] = static_cast<uint8_t*>(desc->g[q]);
    p.r_peer[q] = static_cast<__nv_bfloat16*>(desc->r[q]);
  }
  p.g_local = static_cast<uint8_t*>(desc->g[desc->rank]);
  p.r_local = static_cast<__nv_bfloat16*>(desc->r[desc->rank]);
  p.rows_per_rank = M / n;
  if (desc->scatter && (p.tiles_m / n) * p.tiles_n > JPB_MAX_TILES_PER_RANK) return -JPB_ERR_BAD_ARGUMENT;
  const void* a_ptr = A;
  const void* b_ptr = B;
  const void* own = nullptr;
  int own_width = 0;
  if (desc->gather == GATHER_ROWS) {
    if (a_mn_major || desc->gathered_is_b || !A) return -JPB_ERR_BAD_ARGUMENT;
    own = A;
    own_width = K;
    a_ptr = p.g_local;
    lda = K;
    p.chunks_per_rank = p.tiles_m / n;
    p.rows_per_slot = M / n;
    p.chunk_bytes = (long long)CBM * K * 2;
  } else if (desc->gather == GATHER_RED) {
    own_width = desc->gathered_is_b ? N : M;
    if (desc->gathered_is_b) { if (!b_mn_major || !B) return -JPB_ERR_BAD_ARGUMENT; own = B; b_ptr = p.g_local; ldb = N; }
    else { if (!a_mn_major || !A) return -JPB_ERR_BAD_ARGUMENT; own = A; a_ptr = p.g_local; lda = M; }
    p.chunks_per_rank = (K / CBK) / n;
    p.rows_per_slot = K / n;
    p.chunk_bytes = (long long)CBK * own_width * 2;
    if (out_fp32 && !desc->scatter) p.phases = n;
  }
  if (desc->gather) {
    if (n * p.chunks_per_rank > JPB_MAX_CHUNKS || (own_width & 7)) return -JPB_ERR_BAD_ARGUMENT;
    p.piece_bytes = p.chunk_bytes < PIECE_BYTES ? p.chunk_bytes : PIECE_BYTES;
    p.pieces = int((p.chunk_bytes + p.piece_bytes - 1) / p.piece_bytes);
    p.own_src = static_cast<const uint8_t*>(own);
    p.gather_out = static_cast<uint8_t*>(gather_out);
    if ((reinterpret_cast<uintptr_t>(own) & 15) || (reinterpret_cast<uintptr_t>(gather_out) & 15)) return -JPB_ERR_BAD_ARGUMENT;
  }
  if ((reinterpret_cast<uintptr_t>(a_ptr) & 15) || (reinterpret_cast<uintptr_t>(b_ptr) & 15) || (lda & 7) || (ldb & 7))
    return -JPB_ERR_BAD_ARGUMENT;
  CUtensorMap ma, mb, mo;
  p.a_blocked = a_mn_major && M % 64 == 0;
  p.b_blocked = b_mn_major && N % 64 == 0;
  int rc;
  if (!a_mn_major) rc = comm_map_2d(&ma, a_ptr, K, M, lda, CBK, CBM);
  else if (p.a_blocked) rc = comm_map_mn_blocked(&ma, a_ptr, M, K, lda, CBM / 64);
  else rc = comm_map_2d(&ma, a_ptr, M, K, lda, 64, CBK);
  if (rc) return rc;
  if (!b_mn_major) rc = comm_map_2d(&mb, b_ptr, K, N, ldb, CBK, CBN);
  else if (p.b_blocked) rc = comm_map_mn_blocked(&mb, b_ptr, N, K, ldb, CBN / 64);
  else rc = comm_map_2d(&mb, b_ptr, N, K, ldb, 64, CBK);
  if (rc) return rc;
  if (desc->gather == GATHER_ROWS) {
    rc = comm_map_2d(&mo, own, K, p.rows_per_slot, K, CBK, CBM);
  } else if (desc->gather == GATHER_RED) {
    const bool blocked = desc->gathered_is_b ? p.b_blocked : p.a_blocked;
    const uint32_t blocks = desc->gathered_is_b ? CBN / 64 : CBM / 64;
    rc = blocked ? comm_map_mn_blocked(&mo, own, own_width, p.rows_per_slot, own_width, blocks)
                 : comm_map_2d(&mo, own, own_width, p.rows_per_slot, own_width, 64, CBK);
  } else {
    mo = ma;
  }
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn_major && !b_mn_major) return comm_launch<false, false>(ma, mb, mo, p, desc->max_ctas, s);
  if (!a_mn_major && b_mn_major) return comm_launch<false, true>(ma, mb, mo, p, desc->max_ctas, s);
  if (a_mn_major && b_mn_major) return comm_launch<true, true>(ma, mb, mo, p, desc->max_ctas, s);
  return comm_launch<true, false>(ma, mb, mo, p, desc->max_ctas, s);
}
