// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a).
//
// One persistent kernel per op; the tcgen05 main loop is the one of gemm_sm100.cu (TMA ring -> tcgen05.mma
// -> double-buffered TMEM accumulators -> epilogue warps) plus a seventh "comm" warp per CTA.
//
//  all-gather -> GEMM   The gathered operand lives in a symmetric buffer G[n_ranks][rows_per_rank, width]
//                       that exists on every rank; a rank's own slot is filled before the launch.  Comm
//                       warps pull the peers' slots over NVLink (plain 16-byte peer loads, each byte crosses
//                       the link once) into the local copy of G chunk by chunk and publish a flag per chunk;
//                       the TMA producer runs the tiles (or k-blocks) that depend only on the local slot
//                       first and waits on the chunk flag before it touches a pulled chunk.  The gather can
//                       be along the rows of A (forward / dgrad) or along the reduction dimension (wgrad).
//  GEMM -> reduce-scatter
//                       Output row block p belongs to rank p.  Tiles of the peers' blocks are computed first;
//                       their epilogue stores the bf16 partial tile straight into the owner's receive buffer
//                       (peer stores) and then raises a per-tile flag in the owner's memory.  Tiles of the own
//                       block run last; their epilogue waits for the peers' flags, adds the received partials
//                       in fp32 and writes the final tile.
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
constexpr int COMM_THREADS = 224;  // TMA, MMA, 4 epilogue warps, comm warp
constexpr int CSMEM_BYTES = CSTAGES * CSTAGE_BYTES + 1024 + 256;
constexpr int MAX_RANKS = 8;

enum GatherMode : int { GATHER_NONE = 0, GATHER_ROWS = 1, GATHER_RED = 2 };

struct CommGemmParams {
  int M, N, K;
  int ldd, out_fp32, accumulate, bias_fp32;
  const void* bias;
  void* D;
  int* status;
  int tiles_m, tiles_n;
  // --- collective ---
  int n_ranks, rank;
  int epoch;                         // > 0, increases with every call on this workspace
  // all-gather
  int gather;                        // GatherMode
  int chunks_per_rank;               // m-tiles (GATHER_ROWS) or k-blocks (GATHER_RED) per rank slot
  long long chunk_bytes;             // contiguous bytes of one chunk inside G
  uint8_t* g_local;                  // this rank's G
  const uint8_t* g_peer[MAX_RANKS];  // every rank's G as mapped here (g_peer[rank] == g_local)
  int* chunk_flags;                  // local, [n_ranks * chunks_per_rank]
  int* ready_local;                  // local, [n_ranks]: ready_local[p] == epoch  <=> peer p's own slot is valid
  int* ready_peer[MAX_RANKS];        // the same array in every peer's memory
  // reduce-scatter
  int scatter;                       // 0/1
  __nv_bfloat16* r_local;            // receive buffer [n_ranks][rows_per_rank, N] (slot = source rank)
  __nv_bfloat16* r_peer[MAX_RANKS];
  int* tile_flags_local;             // [n_ranks][tiles_m_per_rank * tiles_n]
  int* tile_flags_peer[MAX_RANKS];
  int rows_per_rank;                 // M / n_ranks for scatter
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Spin until *flag >= want (flags only grow), at most JPB_WAIT_BUDGET_NS.  `sys` selects the scope of the load.
__device__ __forceinline__ bool flag_wait_bounded(const int* flag, int want, bool sys, volatile int* abort_flag, int* status,
                                                  int code) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (true) {
    const int v = sys ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
    if (v >= want) return true;
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > JPB_WAIT_BUDGET_NS) {
        *abort_flag = 1;
        if (status) atomicCAS(status, JPB_OK, code);
        return false;
      }
    }
  }
}

// Tile order: with a scatter, the row blocks of the peers come first (starting with the next rank) and the
// own block last; with a row gather, the own block comes first.  Inside a row block tiles are m-fastest.
struct TileOrder {
  int tiles_m, tiles_n, n_ranks, rank, tm_per_rank, mode;  // mode: 0 plain, 1 own-first, 2 own-last
  __device__ __forceinline__ void get(int idx, int& m_blk, int& n_blk) const {
    // inside a row block tiles are walked in groups of 16 row tiles, column by column (L2-friendly)
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
    const int shift = mode == 1 ? blk : blk + 1;
    const int slot = (rank + shift) % n_ranks;
    m_blk = slot * tm_per_rank + lm;
  }
};

__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(COMM_THREADS, 1)
comm_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const CommGemmParams p, int* done_counter, long long counter_target) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + CSTAGES * CSTAGE_BYTES);
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

  if (threadIdx.x == 0) {
    for (int s = 0; s < CSTAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    mbar_init(epi_bar, 4);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (blockIdx.x == 0 && p.gather != GATHER_NONE) {
      // this rank's own slot of G was filled before the launch: tell every peer it may be pulled
      for (int q = 0; q < p.n_ranks; ++q)
        if (q != p.rank) st_release_sys(p.ready_peer[q] + p.rank, p.epoch);
    }
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
      bool all_pulled = p.gather == GATHER_NONE;
      auto chunk_ready = [&](int chunk) -> bool {
        if (all_pulled) return true;
        if (chunk / p.chunks_per_rank == p.rank) return true;
        if (!flag_wait_bounded(p.chunk_flags + chunk, p.epoch, false, abort_flag, p.status, JPB_ERR_PEER_TIMEOUT)) return false;
        if ((long long)ld_acquire_gpu(done_counter) >= counter_target) all_pulled = true;
        fence_proxy_async_global();
        return true;
      };
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        order.get(tile, m_blk, n_blk);
        const int m0 = m_blk * CBM, n0 = n_blk * CBN;
        if (p.gather == GATHER_ROWS && !chunk_ready(m_blk)) { ok = false; break; }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int kbe = (kb + k_rot) % k_blocks;
          if (p.gather == GATHER_RED && !chunk_ready(kbe)) { ok = false; break; }
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
            tma_load_2d(sa, &map_a, &full[s], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < CBM / 64; ++j) tma_load_2d(sa + j * 8192, &map_a, &full[s], m0 + j * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d(sb, &map_b, &full[s], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < CBN / 64; ++j) tma_load_2d(sb + j * 8192, &map_b, &full[s], n0 + j * 64, k0);
          }
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        for (int s = 0; s < CSTAGES; ++s) {
          if (!(armed & (1u << s))) continue;
          while (!mbar_try_wait(&full[s], (armed_phase >> s) & 1) && globaltimer_ns() - t0 < JPB_WAIT_BUDGET_NS) {
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
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_i) {
        const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait_bounded(&acc_empty[acc], acc_ph ^ 1, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * CBN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
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
  } else if (warp == 6) {
    // ------------------------------------------ comm warp: pull peers' slots ----------------------------
    if (p.gather != GATHER_NONE) {
      const int remote_chunks = (p.n_ranks - 1) * p.chunks_per_rank;
      int ready_seen = 0;  // bit q set once peer q announced its slot
      bool ok = true;
      for (int idx = blockIdx.x; idx < remote_chunks && ok; idx += gridDim.x) {
        const int slot = (p.rank + 1 + idx / p.chunks_per_rank) % p.n_ranks;
        const int chunk = slot * p.chunks_per_rank + idx % p.chunks_per_rank;
        if (!(ready_seen & (1 << slot))) {
          bool w = flag_wait_bounded(p.ready_local + slot, p.epoch, true, abort_flag, p.status, JPB_ERR_PEER_TIMEOUT);
          w = __all_sync(0xffffffffu, w);
          if (!w) { ok = false; break; }
          ready_seen |= 1 << slot;
        }
        const uint8_t* src = p.g_peer[slot] + (long long)chunk * p.chunk_bytes;
        uint8_t* dst = p.g_local + (long long)chunk * p.chunk_bytes;
        const long long nvec = p.chunk_bytes / 16;
        long long v = lane;
        for (; v + 7 * 32 < nvec; v += 8 * 32) {
          uint4 r[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) r[u] = ld_volatile_v4(src + (v + u * 32) * 16);
#pragma unroll
          for (int u = 0; u < 8; ++u) *reinterpret_cast<uint4*>(dst + (v + u * 32) * 16) = r[u];
        }
        for (; v < nvec; v += 32) *reinterpret_cast<uint4*>(dst + v * 16) = ld_volatile_v4(src + v * 16);
        __threadfence();
        fence_proxy_async_global();
        __syncwarp();
        if (lane == 0) {
          st_release_gpu(p.chunk_flags + chunk, p.epoch);
          atomicAdd(done_counter, 1);
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
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_i) {
      int m_blk, n_blk;
      order.get(tile, m_blk, n_blk);
      const int m0 = m_blk * CBM, n0 = n_blk * CBN;
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
        bool w = true;
        for (int q = 0; q < p.n_ranks && w; ++q) {
          if (q == p.rank) continue;
          w = flag_wait_bounded(p.tile_flags_local + q * tiles_per_rank + lm * p.tiles_n + n_blk, p.epoch, true, abort_flag,
                                p.status, JPB_ERR_PEER_TIMEOUT);
        }
        w = __all_sync(0xffffffffu, w);
        if (!w) { ok = false; break; }
      }
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
        if (remote) {
          __nv_bfloat16* d = p.r_peer[owner] + (size_t(p.rank) * p.rows_per_rank + local_row) * p.N + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (j < ncols) {
              uint4 o;
              o.x = pack_bf16(v[j], v[j + 1]); o.y = pack_bf16(v[j + 2], v[j + 3]);
              o.z = pack_bf16(v[j + 4], v[j + 5]); o.w = pack_bf16(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(d + j) = o;
            }
          }
          continue;
        }
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
        if (p.bias) {
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
              if (p.accumulate) {
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

// 2-D bf16 tensor map (row-major, `cols` contiguous)
static int comm_map_2d(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t ld_elems, uint32_t box_cols,
                       uint32_t box_rows) {
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {ld_elems * 2};
  uint32_t box[2] = {box_cols, box_rows};
  return jpb_make_tensor_map(out, base, 2, 2, dims, strides, box, 1);
}

template <bool A_MN, bool B_MN>
static int comm_launch(const CUtensorMap& ma, const CUtensorMap& mb, const CommGemmParams& p, int* counter, long long target,
                       cudaStream_t stream) {
  auto kernel = comm_gemm_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CSMEM_BYTES) != cudaSuccess) return -3;
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // The grid must be fully co-resident: comm warps of every CTA make progress while producers wait on them.
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sms ? tiles : sms;
  kernel<<<grid, COMM_THREADS, CSMEM_BYTES, stream>>>(ma, mb, p, counter, target);
  return int(cudaGetLastError());
}

}  // namespace jpb

// Layout of the per-rank control block (ints) inside the symmetric workspace.
#define JPB_CTRL_READY 0          /* [8]  */
#define JPB_CTRL_COUNTER 8        /* [1]  */
#define JPB_CTRL_CHUNK_FLAGS 16   /* [JPB_MAX_CHUNKS] */
#define JPB_MAX_CHUNKS 4096
#define JPB_CTRL_TILE_FLAGS (16 + JPB_MAX_CHUNKS) /* [8 * JPB_MAX_TILES_PER_RANK] */
#define JPB_MAX_TILES_PER_RANK 8192
#define JPB_CTRL_INTS (JPB_CTRL_TILE_FLAGS + 8 * JPB_MAX_TILES_PER_RANK)

struct JpbCommDesc {
  int n_ranks, rank, epoch;
  int gather;            // 0 none, 1 rows of A, 2 reduction dimension
  int gathered_is_b;     // which operand is read from G (its pointer argument is ignored)
  int scatter;
  long long counter_target;
  void* ctrl[8];         // control block of every rank as mapped in this process
  void* g[8];            // gather buffer (current parity) of every rank
  void* r[8];            // receive buffer (current parity) of every rank
};

JPB_API long long jpb_comm_ctrl_bytes() { return (long long)JPB_CTRL_INTS * 4; }

// D = A * B^T with a fused all-gather of one operand and/or reduce-scatter of the output (see file header).
// For gather != 0 the gathered operand is G of shape [n_ranks * rows_per_rank, width] (bf16, contiguous):
//   gather == 1: A = G is [M, K] K-major;  gather == 2: the gathered operand is MN-major, G is [K, M] or [K, N].
// For scatter != 0, D is this rank's [M / n_ranks, N] block.
JPB_API int jpb_comm_gemm(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int lda, int ldb,
                          int ldd, int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int bias_fp32,
                          const JpbCommDesc* desc, void* stream) {
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
  p.gather = desc->gather; p.scatter = desc->scatter;
  int* my_ctrl = static_cast<int*>(desc->ctrl[desc->rank]);
  p.ready_local = my_ctrl + JPB_CTRL_READY;
  p.chunk_flags = my_ctrl + JPB_CTRL_CHUNK_FLAGS;
  p.tile_flags_local = my_ctrl + JPB_CTRL_TILE_FLAGS;
  for (int q = 0; q < n; ++q) {
    int* c = static_cast<int*>(desc->ctrl[q]);
    p.ready_peer[q] = c + JPB_CTRL_READY;
    p.tile_flags_peer[q] = c + JPB_CTRL_TILE_FLAGS;
    p.g_peer[q] = static_cast<const uint8_t*>(desc->g[q]);
    p.r_peer[q] = static_cast<__nv_bfloat16*>(desc->r[q]);
  }
  p.g_local = static_cast<uint8_t*>(desc->g[desc->rank]);
  p.r_local = static_cast<__nv_bfloat16*>(desc->r[desc->rank]);
  p.rows_per_rank = M / n;
  if (desc->scatter && (p.tiles_m / n) * p.tiles_n > JPB_MAX_TILES_PER_RANK) return -JPB_ERR_BAD_ARGUMENT;
  const void* a_ptr = A;
  const void* b_ptr = B;
  if (desc->gather == GATHER_ROWS) {
    if (a_mn_major || desc->gathered_is_b) return -JPB_ERR_BAD_ARGUMENT;
    a_ptr = p.g_local;
    lda = K;
    p.chunks_per_rank = p.tiles_m / n;
    p.chunk_bytes = (long long)CBM * K * 2;
  } else if (desc->gather == GATHER_RED) {
    const int width = desc->gathered_is_b ? N : M;
    if (desc->gathered_is_b) { if (!b_mn_major) return -JPB_ERR_BAD_ARGUMENT; b_ptr = p.g_local; ldb = N; }
    else { if (!a_mn_major) return -JPB_ERR_BAD_ARGUMENT; a_ptr = p.g_local; lda = M; }
    p.chunks_per_rank = (K / CBK) / n;
    p.chunk_bytes = (long long)CBK * width * 2;
  }
  if (desc->gather && n * p.chunks_per_rank > JPB_MAX_CHUNKS) return -JPB_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(a_ptr) & 15) || (reinterpret_cast<uintptr_t>(b_ptr) & 15) || (lda & 7) || (ldb & 7))
    return -JPB_ERR_BAD_ARGUMENT;
  CUtensorMap ma, mb;
  int rc = a_mn_major ? comm_map_2d(&ma, a_ptr, M, K, lda, 64, CBK) : comm_map_2d(&ma, a_ptr, K, M, lda, CBK, CBM);
  if (rc) return rc;
  rc = b_mn_major ? comm_map_2d(&mb, b_ptr, N, K, ldb, 64, CBK) : comm_map_2d(&mb, b_ptr, K, N, ldb, CBK, CBN);
  if (rc) return rc;
  int* counter = my_ctrl + JPB_CTRL_COUNTER;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn_major && !b_mn_major) return comm_launch<false, false>(ma, mb, p, counter, desc->counter_target, s);
  if (!a_mn_major && b_mn_major) return comm_launch<false, true>(ma, mb, p, counter, desc->counter_target, s);
  if (a_mn_major && b_mn_major) return comm_launch<true, true>(ma, mb, p, counter, desc->counter_target, s);
  return comm_launch<true, false>(ma, mb, p, counter, desc->counter_target, s);
}
