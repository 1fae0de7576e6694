// Grouped FP8 GEMM for B200 (sm_100a): persistent, warp-specialised tcgen05 / TMEM kernel.
//
// Replaces the reference's CUTLASS Sm90 grouped GEMM (csrc/fp8_gmm.cu:46-80,82-161), its separate
// de-scale pass (csrc/multi_pointwise.cu:99-151) and the per-group cuBLASLt loops (fp8_gmm/backend.py:
// 84-96; wgrad: fp8_gmm/grouped_linear.py:165-182) with one launch per GEMM.
//
// Kernel shape
//   * one persistent CTA per SM, 192 threads: warp 0 = TMA producer, warp 1 = MMA issuer (and TMEM
//     owner), warps 2-5 = epilogue (each owns the 32 TMEM lanes its warp id selects);
//   * output tile 128 x 256 per CTA, or 256 x 256 per CTA pair (cta_group::2, the default for large groups);
//     K step 128 bytes (one 128-byte swizzle atom); shared-memory ring of 4 stages x 48 KiB (single CTA) or
//     6 stages x 32 KiB (pair: every CTA loads its own 128 A rows and 128 B rows), K-major, written by TMA
//     with SWIZZLE_128B;
//   * tcgen05.mma.cta_group::1.kind::f8f6f4, M=128 N=256 K=32, fp32 accumulators in TMEM; the 512 TMEM
//     columns hold two accumulators so the epilogue of tile i overlaps the main loop of tile i+1;
//   * epilogue: tcgen05.ld -> (a_scale_inv*b_scale_inv) -> bf16; full 32-row slabs are staged in shared memory
//     (SWIZZLE_128B boxes) and written by TMA stores, slabs that straddle the end of their group fall back to
//     predicated 16-byte stores; optional fused activation (GELU or SwiGLU) that also emits the e4m3
//     activation and its amax;
//   * device-side scheduler: every role walks the same static tile sequence blockIdx.x + i*gridDim.x and
//     decodes (group, m-tile, n-tile) from prefix sums held in the kernel parameter block.  Tiles are
//     ordered group-major and, inside a group, in super-rows of 4096 rows (2048 for long contractions) with
//     m fastest, so the concurrently running tiles share operand tiles through L2;
//   * no multicast: every CTA loads its own operands.  (Asking the TMA unit to prefetch the K block 8-16 steps ahead
//     into L2 was measured 10 % slower, whether every CTA prefetched its boxes or one CTA per distinct box did: the
//     extra requests cost the TMA queue more than the shorter fill latency gives back.)
// Two addressing modes share the kernel: "rows" (forward/dgrad: groups are row blocks of one A matrix,
// B is (G,N,K)) and "wgrad" (each group has its own pair of TMA descriptors in global memory because the
// padded-transposed operand blocks have a group-dependent row pitch; contraction length varies per group).
//
// Every wait on an mbarrier is bounded (about one second of wall clock); when it runs out the CTA
// records a code in the device status word, raises a CTA-wide abort flag that all roles poll, drains and
// frees its TMEM, and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace fp8gmm {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 128;  // bytes == fp8 elements
// Tile order inside a group: super-rows of this many rows, m fastest inside a super-row.  With a short
// contraction a 4096-row band of A stays in L2 while the n-tiles sweep past it, so A and B are each read from
// DRAM about once (measured: 1.10 GB for 1.07 GB of operands, N = 28672, K = 4096).  With a long contraction
// neither band fits, reuse only happens among the ~74 tiles in flight, and a squarer wave (8 x 9 tiles rather
// than 16 x 4.6) touches fewer distinct operand rows.
constexpr int kSuperRowsShortK = 4096;
constexpr int kSuperRowsLongK = 2048;
constexpr int kLongK = 8192;
constexpr int kThreads = 192;
constexpr int kTileABytes = kBlockM * kBlockK;          // 16 KiB
constexpr int kTileBBytes = kBlockN * kBlockK;          // 32 KiB
constexpr int kTmemCols = 512;
constexpr int kMaxGroups = 512;

enum GemmMode { kModeRows = 0, kModeWgrad = 1 };
// Row map entries that name a destination rank (GemmParams::c_peers): rank in the bits from kPeerShift up, row below.
constexpr int kPeerShift = FP8GMM_ROW_MAP_PEER_SHIFT;
constexpr int kPeerRowMask = (1 << kPeerShift) - 1;

struct GemmParams {
  CUtensorMap map_a;          // kModeRows: A (sum m, K)
  CUtensorMap map_b;          // kModeRows: B (G*N, K)
  CUtensorMap map_c;          // bf16 result (or pre-activation) as a 2-D tensor, box 64 columns x 32 rows, for TMA stores
  const CUtensorMap* maps;    // kModeWgrad: [2g] = A_t,g (N, L_g), [2g+1] = B_t,g (K, L_g)
  uint16_t* c;
  uint8_t* act_out;
  const uint16_t* aux_in;  // FP8GMM_ACT_DSWIGLU: bf16 pre-activation [gate | up], (sum m x 2n)
  const float* sa;
  const float* sb;
  const float* sc;
  float* amax;
  int64_t sa_stride, sb_stride, sc_stride, amax_stride;
  int64_t ldc;     // row pitch of c in elements
  int64_t ld_act;  // row pitch of act_out in bytes
  int* status;
  const int32_t* row_map;  // optional (plain epilogue, rows mode): output row r is stored at row row_map[r] of c
  const unsigned long long* c_peers;  // optional, with row_map: base addresses of the ranks' result buffers; a map entry
                                      // is then (rank << kPeerShift) | row and the row is stored in that rank's buffer
  unsigned long long wait_ns;  // limit of every mbarrier wait (fp8gmm_set_wait_limits)
  unsigned int* wave_counter;  // long contractions: tiles started so far (zeroed before the launch), or NULL
  int b_mn;            // kModeRows only: B is (G, K, N) row-major, read MN-major through the 3-D map_b (x = n, y = k, z = group)
  int mn_major;        // kModeWgrad only: operands are row-major (rows x features) slices, i.e. MN-major for the MMA
  int super_tiles;     // m-tiles per super-row of the tile order (see decode_tile)
  int tma_store;       // 1: full 32-row slabs of a tile leave through shared memory + TMA stores (map_c is valid)
  int mode;
  int activation;
  int act_format;      // fp8 format of act_out (the forward activations are e4m3, the fused backward writes e5m2 or e4m3)
  int num_groups;
  int n;        // kModeRows: N (columns of C); kModeWgrad: K-dim of the weight (columns of C_g)
  int m_fixed;  // kModeWgrad: rows of every C_g (= N of the layer)
  int k;        // kModeRows: contraction length
  int tiles_n;  // n-tiles per group
  int total_tiles;
  uint32_t idesc;
  int tile_start[kMaxGroups + 1];  // prefix sum of tiles per group
  int row_start[kMaxGroups + 1];   // kModeRows: first row of the group's slice; kModeWgrad: t_offsets (contraction offsets)
  int row_count[kMaxGroups];       // kModeRows: rows of the group this launch covers (a launch may leave a tail to another)
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait.  Returns false (after raising the CTA abort flag and recording `code`) when the barrier
// did not complete its phase within `limit_ns`, or when another role already aborted.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                            unsigned long long limit_ns) {
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > limit_ns) {
      *abort_flag = 1;
      atomicOr(status, code);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, code, limit_ns);
}

// Soft wave barrier for long contractions.  The tiles that run side by side share operand boxes through L2 (an A box
// is read by every n-tile in flight, a B box by every m-tile of the super-row), which only works while they sweep the
// contraction in step.  With a contraction of 14336 or 28672 a tile takes ~100 us, the CTA pairs drift apart by more
// than L2 can bridge, and DRAM reads grow to several times the operand bytes.  So before its first load of a tile the
// leader's producer counts itself in and waits until every tile of the same wave has been started -- for at most
// kWaveWaitNs: this is a hint, not a dependency, and a pair that is late (or not yet resident) is simply not waited for.
constexpr unsigned long long kWaveWaitNs = 20000ull;
__device__ __forceinline__ void wave_arrive_and_wait(unsigned int* counter, unsigned int target) {
  atomicAdd(counter, 1u);
  const unsigned long long t0 = global_ns();
  while (*reinterpret_cast<volatile unsigned int*>(counter) < target) {
    if (global_ns() - t0 > kWaveWaitNs) break;
    __nanosleep(100);
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// A tensor map that lives in global memory and was written through the generic proxy (here: by a host-to-device
// copy that precedes the kernel on its stream) must be acquired by the thread that hands it to the TMA unit before
// its first use; system scope because the writer was not this GPU's SMs.
__device__ __forceinline__ void acquire_tensormap(const CUtensorMap* map) {
  asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- TMA store of a staged (32 rows x 128 bytes, SWIZZLE_128B) box -------------------------------
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once at most kPending of this thread's bulk groups still read their shared-memory source.
template <int kPending>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Orders this thread's generic-proxy shared-memory writes before later async-proxy (TMA) reads of them.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void st_shared16(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_shared16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// Byte offset of 16-byte chunk `c` (0..7) of row `r` (0..31) inside a 4 KiB staging box with 128-byte rows in
// the SWIZZLE_128B pattern the tensor map expects (the box starts on a 1024-byte boundary).
__device__ __forceinline__ uint32_t staged_chunk(int r, int c) { return static_cast<uint32_t>(r * 128 + ((c ^ (r & 7)) << 4)); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread = lane = row).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile written by TMA with SWIZZLE_128B:
// rows are 128 bytes apart inside an 8-row swizzle atom, atoms are 1024 bytes apart (stride byte
// offset); the leading byte offset is unused for swizzled K-major layouts.  Bits: [0,14) address>>4,
// [16,30) LBO>>4, [32,46) SBO>>4, [46,48) descriptor version (1 on sm_100), [61,64) layout (2 = 128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Shared-memory matrix descriptor for an MN-major operand tile: TMA wrote [contraction rows][128 bytes of the M/N
// dimension] with SWIZZLE_128B, so a swizzle atom is 8 contraction rows x 128 M/N bytes (1024 bytes).  Stride byte
// offset = distance between consecutive 8-row groups along the contraction (1024); leading byte offset = distance
// between consecutive 128-byte blocks along M/N (only used when the operand is wider than 128, i.e. the 256-wide B
// of the single-CTA kernel, whose second block is a second TMA box).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  return 0.5f * x * (1.f + tanhf(0.79788456f * x * (1.f + 0.044715f * x * x)));
}

struct TileInfo {
  int group, mt, nt;
  int num_kb;      // K blocks of 128 bytes
  int valid_rows;  // rows of this CTA's 128-row slab that belong to the output (may be <= 0)
  int valid_cols;
  int64_t row0;    // first output row of this CTA's slab (kModeRows: global row; kModeWgrad: row inside C_g)
};

// kCtas = 1: a CTA owns a 128 x 256 tile.  kCtas = 2: a pair of CTAs (cluster of 2) owns a 256 x 256
// tile, CTA `rank` holding rows [128*rank, 128*rank+128) of it.
template <int kCtas>
__device__ __forceinline__ TileInfo decode_tile(const GemmParams& p, int tile, int rank) {
  constexpr int kTileM = kBlockM * kCtas;
  const int kSuper = p.super_tiles;
  TileInfo t;
  const int g = upper_slot(p.tile_start, p.num_groups, tile);
  const int local = tile - p.tile_start[g];
  int rows_g, contraction;
  if (p.mode == kModeRows) {
    rows_g = p.row_count[g];
    contraction = p.k;
  } else {
    rows_g = p.m_fixed;
    contraction = p.row_start[g + 1] - p.row_start[g];
  }
  const int mt_g = (rows_g + kTileM - 1) / kTileM;
  const int per_super = kSuper * p.tiles_n;
  const int s = local / per_super;
  const int rem = local - s * per_super;
  const int h = min(kSuper, mt_g - s * kSuper);
  t.group = g;
  t.nt = rem / h;
  t.mt = s * kSuper + rem % h;
  t.num_kb = (contraction + kBlockK - 1) / kBlockK;
  const int slab = t.mt * kTileM + rank * kBlockM;
  t.valid_rows = min(kBlockM, rows_g - slab);
  const int tile_n = p.activation == FP8GMM_ACT_SWIGLU ? kBlockN / 2 : kBlockN;
  const int n_cols = p.activation == FP8GMM_ACT_SWIGLU ? p.n / 2 : p.n;
  t.valid_cols = min(tile_n, n_cols - t.nt * tile_n);
  t.row0 = (p.mode == kModeRows ? static_cast<int64_t>(p.row_start[g]) : 0) + slab;
  return t;
}

// ---- cluster helpers (kCtas = 2) ----------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes may be credited to an mbarrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// One MMA over both CTAs of the pair: M = 256 (128 rows from each CTA's A tile and TMEM), N = 256 (128 B rows
// from each CTA's shared memory); issued by one thread of the leader CTA.
__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in both CTAs once all MMAs issued so far are complete.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}

template <int kCtas>
struct Cfg {
  static constexpr int kStages = kCtas == 1 ? 4 : 6;
  static constexpr int kBRows = kBlockN / kCtas;              // B rows held by one CTA
  static constexpr int kBBytes = kBRows * kBlockK;
  static constexpr int kStageBytes = kTileABytes + kBBytes;   // 48 KiB (1 CTA) / 32 KiB (pair)
  static constexpr int kStagingBytes = 4 * 8192;             // per epilogue warp: two 4 KiB boxes for TMA stores
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
template <int kCtas>
__device__ __forceinline__ void gemm_body(const GemmParams& p) {
  using C = Cfg<kCtas>;
  constexpr int kStages = C::kStages;
  constexpr int kStageBytes = C::kStageBytes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;  // SWIZZLE_128B atoms need 1024-byte alignment
  uint8_t* tiles_ptr = smem_raw + (tiles_addr - raw_addr);
  const uint32_t staging_addr = tiles_addr + kStages * kStageBytes;  // 1024-byte aligned: stages are multiples of 1 KiB
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles_ptr + kStages * kStageBytes + C::kStagingBytes);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kStages + 2 + a); };
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = kCtas == 2 ? static_cast<int>(cluster_ctarank()) : 0;
  const bool leader = rank == 0;
  const int worker = kCtas == 2 ? blockIdx.x >> 1 : blockIdx.x;        // tile-sequence index of this CTA (pair)
  const int num_workers = kCtas == 2 ? gridDim.x >> 1 : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4 * kCtas);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (kCtas == 2) {
      tmem_alloc_pair(smem_u32(tmem_base_slot), kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_base_slot), kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if (kCtas == 2) cluster_sync_all(); else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ===================== TMA producer (every CTA loads its own operand slabs) =====================
    // One thread runs the whole loop; the other lanes park at the __syncwarp below.
    if (lane == 0) {
      if (p.mode == kModeRows) {
        prefetch_tensormap(&p.map_a);
        prefetch_tensormap(&p.map_b);
      }
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int acquired_group = -1;
      const uint32_t full0_leader = kCtas == 2 ? map_to_cta(full_bar(0), 0) : 0;
      for (int tile = worker; tile < p.total_tiles && ok; tile += num_workers) {
        const TileInfo t = decode_tile<kCtas>(p, tile, rank);
        if (p.wave_counter != nullptr && leader) {
          const int wave_end = (tile / num_workers + 1) * num_workers;
          wave_arrive_and_wait(p.wave_counter, static_cast<unsigned int>(min(wave_end, p.total_tiles)));
        }
        const CUtensorMap* map_a = p.mode == kModeRows ? &p.map_a : &p.maps[2 * t.group];
        const CUtensorMap* map_b = p.mode == kModeRows ? &p.map_b : &p.maps[2 * t.group + 1];
        if (p.mode == kModeWgrad && t.group != acquired_group && t.num_kb > 0) {
          acquire_tensormap(map_a);
          acquire_tensormap(map_b);
          acquired_group = t.group;
        }
        // first B row of each 128-row box this CTA loads: 1 CTA -> two boxes (columns [0,128) and [128,256) of the
        // tile); pair -> one box, the half selected by `rank`.  SwiGLU: first half = gate rows, second = up rows.
        int yb0, yb1;
        const int b_base = p.mode == kModeRows ? t.group * p.n : 0;
        if (p.activation == FP8GMM_ACT_SWIGLU) {
          yb0 = b_base + t.nt * (kBlockN / 2);
          yb1 = yb0 + p.n / 2;
        } else {
          yb0 = b_base + t.nt * kBlockN;
          yb1 = yb0 + kBlockN / 2;
        }
        const int ya = static_cast<int>(t.row0);
        const int yb_mine = rank == 0 ? yb0 : yb1;
        for (int kb = 0; kb < t.num_kb && ok; ++kb) {
          ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 0x1, p.wait_ns);
          if (ok) {
            const uint32_t sa = tiles_addr + stage * kStageBytes;
            const uint32_t sb = sa + kTileABytes;
            // K-major operands: x = contraction offset, y = operand row.  MN-major (row-major slices of the
            // activations): x = feature offset, y = contraction row; the box is 128 x 128 bytes either way.
            const int kx = kb * kBlockK;
            const bool mn = p.mn_major != 0;
            if (kCtas == 1) {
              mbar_expect_tx(full_bar(stage), kStageBytes);
              tma_load_2d(sa, map_a, full_bar(stage), mn ? ya : kx, mn ? kx : ya);
              if (p.b_mn) {
                // B = (G, K, N): x = output column inside the group, y = contraction row, z = group
                tma_load_3d(sb, map_b, full_bar(stage), yb0 - b_base, kx, t.group);
                tma_load_3d(sb + kTileBBytes / 2, map_b, full_bar(stage), yb1 - b_base, kx, t.group);
              } else {
                tma_load_2d(sb, map_b, full_bar(stage), mn ? yb0 : kx, mn ? kx : yb0);
                tma_load_2d(sb + kTileBBytes / 2, map_b, full_bar(stage), mn ? yb1 : kx, mn ? kx : yb1);
              }
            } else {
              // both CTAs credit the leader's barrier; the leader arms it for the bytes of both
              const uint32_t bar = full0_leader + 8u * stage;
              if (leader) mbar_expect_tx(full_bar(stage), 2 * kStageBytes);
              tma_load_2d_pair(sa, map_a, bar, mn ? ya : kx, mn ? kx : ya);
              if (p.b_mn)
                tma_load_3d_pair(sb, map_b, bar, yb_mine - b_base, kx, t.group);
              else
                tma_load_2d_pair(sb, map_b, bar, mn ? yb_mine : kx, mn ? kx : yb_mine);
            }
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer: one thread (of the leader CTA when paired) =====================
    // The loop is latency critical -- it has to stay ahead of a tensor pipe that retires one K block every
    // 512 cycles -- so it runs in a single thread without warp-level synchronisation inside.
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const bool a_mn = p.mn_major != 0, b_mn = p.mn_major != 0 || p.b_mn != 0;
      const uint64_t desc_a0 = a_mn ? make_smem_desc_mn(tiles_addr, 16) : make_smem_desc(tiles_addr);
      const uint64_t desc_b0 = b_mn ? make_smem_desc_mn(tiles_addr + kTileABytes, kTileBBytes / 2) : make_smem_desc(tiles_addr + kTileABytes);
      // one MMA consumes 32 contraction bytes: 32 bytes along a K-major row, or 32 rows of 128 bytes (MN-major)
      const uint64_t a_step = a_mn ? (32ull * 128ull) >> 4 : 32ull >> 4;
      const uint64_t b_step = b_mn ? (32ull * 128ull) >> 4 : 32ull >> 4;
      const uint32_t idesc = p.idesc;
      for (int tile = worker; tile < p.total_tiles && ok; tile += num_workers) {
        const TileInfo t = decode_tile<kCtas>(p, tile, rank);
        if (t.num_kb == 0) continue;  // empty contraction: the epilogue writes zeros on its own
        ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 0x2, p.wait_ns);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kBlockN);
        for (int kb = 0; kb < t.num_kb; ++kb) {
          ok = mbar_wait(full_bar(stage), phase, abort_flag, p.status, 0x4, p.wait_ns);
          if (!ok) break;
          // descriptors of this stage: the start-address field counts 16-byte units
          const uint64_t da = desc_a0 + static_cast<uint64_t>(stage * (kStageBytes >> 4));
          const uint64_t db = desc_b0 + static_cast<uint64_t>(stage * (kStageBytes >> 4));
#pragma unroll
          for (int k = 0; k < kBlockK / 32; ++k) {
            // advance both descriptors by one MMA's worth of contraction (the steps are in 16-byte units)
            if (kCtas == 1)
              umma_f8(tmem_d, da + a_step * k, db + b_step * k, idesc, (kb | k) != 0 ? 1u : 0u);
            else
              umma_f8_pair(tmem_d, da + a_step * k, db + b_step * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if (kCtas == 1) umma_commit(empty_bar(stage)); else umma_commit_pair(empty_bar(stage));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (kCtas == 1) umma_commit(tfull_bar(acc)); else umma_commit_pair(tfull_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue (warps 2..5) =====================
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may read
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = worker; tile < p.total_tiles && ok; tile += num_workers) {
      const TileInfo t = decode_tile<kCtas>(p, tile, rank);
      const bool row_ok = row_in_tile < t.valid_rows;
      const int64_t out_row = t.row0 + row_in_tile;
      const float alpha = p.sa[t.group * p.sa_stride] * p.sb[t.group * p.sb_stride];
      if (t.num_kb == 0) {
        // nothing was accumulated: the product is exactly zero (wgrad of an empty group)
        if (row_ok) {
          uint16_t* dst = p.c + static_cast<int64_t>(t.group) * p.m_fixed * p.ldc + out_row * p.ldc + t.nt * kBlockN;
          for (int c = 0; c < t.valid_cols; c += 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      if (lane == 0) ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, 0x8, p.wait_ns);
      ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + static_cast<uint32_t>(acc * kBlockN) + (static_cast<uint32_t>(quad * 32) << 16);

      // A warp whose 32 rows all belong to the tile stages its results in shared memory and lets TMA write
      // them (full 128-byte lines per row instead of 32 scattered 16-byte stores per instruction).
      const int tile_cols = p.activation == FP8GMM_ACT_SWIGLU ? kBlockN / 2 : kBlockN;
      bool use_tma = p.tma_store != 0 && t.valid_rows - quad * 32 >= 32 && t.valid_cols == tile_cols;
      const uint32_t stage0 = staging_addr + static_cast<uint32_t>(quad) * 8192u;
      int row_coord = static_cast<int>((p.mode == kModeWgrad ? static_cast<int64_t>(t.group) * p.m_fixed : 0) + t.row0) + quad * 32;
      if (use_tma && p.row_map != nullptr) {
        // A row map moves whole runs of rows (blocks of one expert and one source rank): a slab whose 32 rows stay
        // consecutive at their destination still leaves as TMA boxes, at the mapped row; only slabs that straddle
        // the end of a run take the per-thread stores below.
        const int mine = p.row_map[out_row];
        const int first = __shfl_sync(0xFFFFFFFFu, mine, 0);
        use_tma = __all_sync(0xFFFFFFFFu, mine == first + lane);
        row_coord = first;
      }
      if (p.activation == FP8GMM_ACT_NONE && use_tma) {
        const int col_base = t.nt * kBlockN;
#pragma unroll 1
        for (int c0 = 0; c0 < kBlockN; c0 += 32) {
          const int half = (c0 >> 5) & 1;
          const uint32_t box = stage0 + static_cast<uint32_t>((c0 >> 6) & 1) * 4096u;
          if (half == 0) {
            // the store issued two boxes ago read this buffer: it must be done reading before we overwrite it
            if (lane == 0) bulk_wait_read<1>();
            __syncwarp();
          }
          uint32_t r[32];
          tmem_ld32(taddr + c0, r);
          tc_wait_ld();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]) * alpha, __uint_as_float(r[v * 8 + 1]) * alpha);
            o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]) * alpha, __uint_as_float(r[v * 8 + 3]) * alpha);
            o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]) * alpha, __uint_as_float(r[v * 8 + 5]) * alpha);
            o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]) * alpha, __uint_as_float(r[v * 8 + 7]) * alpha);
            st_shared16(box + staged_chunk(lane, half * 4 + v), o);
          }
          if (half == 1) {
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&p.map_c, box, col_base + c0 - 32, row_coord);
              bulk_commit();
            }
          }
        }
      } else if (p.activation == FP8GMM_ACT_NONE && p.c_peers != nullptr) {
        // The rows leave for their home ranks from here: a map entry names the rank whose buffer takes the row and
        // the row there, and the stores go straight into that rank's memory (plain 16-byte stores through the
        // peer mapping; this rank's own rows take the same path into its own buffer).  A slab whose 32 rows stay
        // consecutive at one destination is staged in shared memory, 64 columns at a time, and written as full
        // 128-byte lines (eight lanes per row, four rows per instruction); a slab that straddles the end of a run
        // of rows stores one row per thread.
        const int entry = row_ok ? p.row_map[out_row] : -1;
        const int first = __shfl_sync(0xFFFFFFFFu, entry, 0);
        const bool slab = first >= 0 && t.valid_cols == kBlockN && __all_sync(0xFFFFFFFFu, entry == first + lane);
        if (slab) {
          uint16_t* base = reinterpret_cast<uint16_t*>(p.c_peers[first >> kPeerShift]) +
                           static_cast<int64_t>(first & kPeerRowMask) * p.ldc + t.nt * kBlockN;
          const int sub_row = lane >> 3, chunk = lane & 7;
#pragma unroll 1
          for (int c0 = 0; c0 < kBlockN; c0 += 64) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t r[32];
              tmem_ld32(taddr + c0 + half * 32, r);
              tc_wait_ld();
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]) * alpha, __uint_as_float(r[v * 8 + 1]) * alpha);
                o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]) * alpha, __uint_as_float(r[v * 8 + 3]) * alpha);
                o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]) * alpha, __uint_as_float(r[v * 8 + 5]) * alpha);
                o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]) * alpha, __uint_as_float(r[v * 8 + 7]) * alpha);
                st_shared16(stage0 + staged_chunk(lane, half * 4 + v), o);
              }
            }
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int rr = it * 4 + sub_row;
              const uint4 o = ld_shared16(stage0 + staged_chunk(rr, chunk));
              *reinterpret_cast<uint4*>(base + static_cast<int64_t>(rr) * p.ldc + c0 + chunk * 8) = o;
            }
            __syncwarp();
          }
        } else {
          uint16_t* dst = row_ok ? reinterpret_cast<uint16_t*>(p.c_peers[entry >> kPeerShift]) +
                                       static_cast<int64_t>(entry & kPeerRowMask) * p.ldc + t.nt * kBlockN
                                 : nullptr;
          for (int c0 = 0; c0 < t.valid_cols; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(taddr + c0, r);
            tc_wait_ld();
            if (row_ok) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                if (c0 + v * 8 < t.valid_cols) {
                  uint4 o;
                  o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]) * alpha, __uint_as_float(r[v * 8 + 1]) * alpha);
                  o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]) * alpha, __uint_as_float(r[v * 8 + 3]) * alpha);
                  o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]) * alpha, __uint_as_float(r[v * 8 + 5]) * alpha);
                  o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]) * alpha, __uint_as_float(r[v * 8 + 7]) * alpha);
                  *reinterpret_cast<uint4*>(dst + c0 + v * 8) = o;
                }
              }
            }
          }
        }
      } else if (p.activation == FP8GMM_ACT_NONE) {
        const int64_t dst_row = (p.row_map != nullptr && row_ok) ? static_cast<int64_t>(p.row_map[out_row]) : out_row;
        uint16_t* dst = p.c + (p.mode == kModeWgrad ? static_cast<int64_t>(t.group) * p.m_fixed * p.ldc : 0) +
                        dst_row * p.ldc + t.nt * kBlockN;
        for (int c0 = 0; c0 < t.valid_cols; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + c0, r);
          tc_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (c0 + v * 8 < t.valid_cols) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]) * alpha, __uint_as_float(r[v * 8 + 1]) * alpha);
                o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]) * alpha, __uint_as_float(r[v * 8 + 3]) * alpha);
                o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]) * alpha, __uint_as_float(r[v * 8 + 5]) * alpha);
                o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]) * alpha, __uint_as_float(r[v * 8 + 7]) * alpha);
                *reinterpret_cast<uint4*>(dst + c0 + v * 8) = o;
              }
            }
          }
        }
      } else if (p.activation == FP8GMM_ACT_DSWIGLU) {
        // SwiGLU backward fused behind the fc2 data-gradient GEMM: the accumulator is d(act) for 256 columns of F;
        // with the forward pre-activation [gate | up] of the same rows and columns it becomes d[gate | up], which is
        // cast to fp8 with the group's scale and stored as the two halves of a (sum m x 2F) matrix, its amax merged.
        // d(act) is rounded to bf16 first, so the values equal what the unfused path (bf16 GEMM output, then the
        // activation-backward cast kernel) computes.  Row per thread: the pre-activation comes in as four 16-byte
        // loads per half and step, issued before the accumulator is read.
        const float sc = p.sc ? p.sc[t.group * p.sc_stride] : 1.f;
        const int64_t ld_pre = 2 * static_cast<int64_t>(p.n);
        const uint16_t* gate = p.aux_in + out_row * ld_pre + t.nt * kBlockN;
        const uint16_t* up = gate + p.n;
        uint8_t* dgate = p.act_out + out_row * p.ld_act + t.nt * kBlockN;
        uint8_t* dup = dgate + p.n;
        const bool e5 = p.act_format == FP8GMM_E5M2;
        float amax = 0.f;
        for (int c0 = 0; c0 < t.valid_cols; c0 += 32) {
          uint4 pg[4], pu[4];
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            pg[v] = pu[v] = make_uint4(0, 0, 0, 0);
            if (row_ok && c0 + v * 8 < t.valid_cols) {
              pg[v] = ld_stream16(gate + c0 + v * 8);
              pu[v] = ld_stream16(up + c0 + v * 8);
            }
          }
          uint32_t r[32];
          tmem_ld32(taddr + c0, r);
          tc_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (c0 + v * 8 < t.valid_cols) {
                const uint32_t gw[4] = {pg[v].x, pg[v].y, pg[v].z, pg[v].w};
                const uint32_t uw[4] = {pu[v].x, pu[v].y, pu[v].z, pu[v].w};
                float v0[8], v1[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  // one bf16 rounding of the de-scaled product, as the unfused GEMM output has
                  const float x = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[v * 8 + j]) * alpha));
                  const float y = (j & 1) ? bf16_hi(gw[j >> 1]) : bf16_lo(gw[j >> 1]);
                  const float z = (j & 1) ? bf16_hi(uw[j >> 1]) : bf16_lo(uw[j >> 1]);
                  const float sg = 1.f / (1.f + __expf(-y));
                  v0[j] = x * z * (sg * (1.f + y * (1.f - sg)));
                  v1[j] = x * (y * sg);
                  amax = fmaxf(fabsf(v0[j]), amax);
                  amax = fmaxf(fabsf(v1[j]), amax);
                }
                uint2 q0, q1;
                if (e5) {
                  q0 = make_uint2(cvt_fp8x4<FP8GMM_E5M2>(sc * v0[0], sc * v0[1], sc * v0[2], sc * v0[3]),
                                  cvt_fp8x4<FP8GMM_E5M2>(sc * v0[4], sc * v0[5], sc * v0[6], sc * v0[7]));
                  q1 = make_uint2(cvt_fp8x4<FP8GMM_E5M2>(sc * v1[0], sc * v1[1], sc * v1[2], sc * v1[3]),
                                  cvt_fp8x4<FP8GMM_E5M2>(sc * v1[4], sc * v1[5], sc * v1[6], sc * v1[7]));
                } else {
                  q0 = make_uint2(cvt_fp8x4<FP8GMM_E4M3>(sc * v0[0], sc * v0[1], sc * v0[2], sc * v0[3]),
                                  cvt_fp8x4<FP8GMM_E4M3>(sc * v0[4], sc * v0[5], sc * v0[6], sc * v0[7]));
                  q1 = make_uint2(cvt_fp8x4<FP8GMM_E4M3>(sc * v1[0], sc * v1[1], sc * v1[2], sc * v1[3]),
                                  cvt_fp8x4<FP8GMM_E4M3>(sc * v1[4], sc * v1[5], sc * v1[6], sc * v1[7]));
                }
                *reinterpret_cast<uint2*>(dgate + c0 + v * 8) = q0;
                *reinterpret_cast<uint2*>(dup + c0 + v * 8) = q1;
              }
            }
          }
        }
        if (p.amax) {
          amax = warp_max(amax);
          if (lane == 0) atomic_max_nonneg(p.amax + t.group * p.amax_stride, amax);
        }
      } else if (p.activation == FP8GMM_ACT_GELU) {
        const float sc = p.sc ? p.sc[t.group * p.sc_stride] : 1.f;
        uint16_t* dst = p.c + out_row * p.ldc + t.nt * kBlockN;
        uint8_t* adst = p.act_out + out_row * p.ld_act + t.nt * kBlockN;
        float amax = 0.f;
        for (int c0 = 0; c0 < t.valid_cols; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + c0, r);
          tc_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (c0 + v * 8 < t.valid_cols) {
                float h[8], g[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  h[j] = __uint_as_float(r[v * 8 + j]) * alpha;
                  g[j] = gelu_tanh(h[j]);
                  amax = fmaxf(amax, fabsf(g[j]));
                }
                *reinterpret_cast<uint4*>(dst + c0 + v * 8) =
                    make_uint4(pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]), pack_bf16x2(h[4], h[5]), pack_bf16x2(h[6], h[7]));
                *reinterpret_cast<uint2*>(adst + c0 + v * 8) =
                    make_uint2(cvt_fp8x4<FP8GMM_E4M3>(g[0] * sc, g[1] * sc, g[2] * sc, g[3] * sc),
                               cvt_fp8x4<FP8GMM_E4M3>(g[4] * sc, g[5] * sc, g[6] * sc, g[7] * sc));
              }
            }
          }
        }
        if (p.amax) {
          amax = warp_max(amax);
          if (lane == 0) atomic_max_nonneg(p.amax + t.group * p.amax_stride, amax);
        }
      } else if (use_tma) {
        // SwiGLU, full slab: gate and up pre-activations leave through TMA (one 64-column box each per two
        // iterations), the e4m3 activation (a fifth of the bytes) through 8-byte stores.
        const float sc = p.sc ? p.sc[t.group * p.sc_stride] : 1.f;
        const int half_n = p.n / 2;
        const int64_t out_row = t.row0 + row_in_tile;
        uint8_t* adst = p.act_out + out_row * p.ld_act + t.nt * (kBlockN / 2);
        const int col_base = t.nt * (kBlockN / 2);
        float amax = 0.f;
#pragma unroll 1
        for (int c0 = 0; c0 < kBlockN / 2; c0 += 32) {
          const int half = (c0 >> 5) & 1;
          if (half == 0) {
            if (lane == 0) bulk_wait_read<0>();  // both boxes are rewritten below
            __syncwarp();
          }
          uint32_t rg[32], ru[32];
          tmem_ld32(taddr + c0, rg);
          tmem_ld32(taddr + kBlockN / 2 + c0, ru);
          tc_wait_ld();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float hg[8], hu[8], a[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              hg[j] = __uint_as_float(rg[v * 8 + j]) * alpha;
              hu[j] = __uint_as_float(ru[v * 8 + j]) * alpha;
              a[j] = hg[j] / (1.f + __expf(-hg[j])) * hu[j];
              amax = fmaxf(amax, fabsf(a[j]));
            }
            st_shared16(stage0 + staged_chunk(lane, half * 4 + v),
                        make_uint4(pack_bf16x2(hg[0], hg[1]), pack_bf16x2(hg[2], hg[3]), pack_bf16x2(hg[4], hg[5]), pack_bf16x2(hg[6], hg[7])));
            st_shared16(stage0 + 4096u + staged_chunk(lane, half * 4 + v),
                        make_uint4(pack_bf16x2(hu[0], hu[1]), pack_bf16x2(hu[2], hu[3]), pack_bf16x2(hu[4], hu[5]), pack_bf16x2(hu[6], hu[7])));
            *reinterpret_cast<uint2*>(adst + c0 + v * 8) =
                make_uint2(cvt_fp8x4<FP8GMM_E4M3>(a[0] * sc, a[1] * sc, a[2] * sc, a[3] * sc),
                           cvt_fp8x4<FP8GMM_E4M3>(a[4] * sc, a[5] * sc, a[6] * sc, a[7] * sc));
          }
          if (half == 1) {
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&p.map_c, stage0, col_base + c0 - 32, row_coord);
              tma_store_2d(&p.map_c, stage0 + 4096u, half_n + col_base + c0 - 32, row_coord);
              bulk_commit();
            }
          }
        }
        if (p.amax) {
          amax = warp_max(amax);
          if (lane == 0) atomic_max_nonneg(p.amax + t.group * p.amax_stride, amax);
        }
      } else {  // SwiGLU: accumulator columns [0,128) = gate, [128,256) = up for the same 128 outputs
        const float sc = p.sc ? p.sc[t.group * p.sc_stride] : 1.f;
        const int half_n = p.n / 2;
        uint16_t* dst_g = p.c + out_row * p.ldc + t.nt * (kBlockN / 2);
        uint16_t* dst_u = dst_g + half_n;
        uint8_t* adst = p.act_out + out_row * p.ld_act + t.nt * (kBlockN / 2);
        float amax = 0.f;
        for (int c0 = 0; c0 < t.valid_cols; c0 += 32) {
          uint32_t rg[32], ru[32];
          tmem_ld32(taddr + c0, rg);
          tmem_ld32(taddr + kBlockN / 2 + c0, ru);
          tc_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (c0 + v * 8 < t.valid_cols) {
                float hg[8], hu[8], a[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  hg[j] = __uint_as_float(rg[v * 8 + j]) * alpha;
                  hu[j] = __uint_as_float(ru[v * 8 + j]) * alpha;
                  a[j] = hg[j] / (1.f + __expf(-hg[j])) * hu[j];
                  amax = fmaxf(amax, fabsf(a[j]));
                }
                *reinterpret_cast<uint4*>(dst_g + c0 + v * 8) =
                    make_uint4(pack_bf16x2(hg[0], hg[1]), pack_bf16x2(hg[2], hg[3]), pack_bf16x2(hg[4], hg[5]), pack_bf16x2(hg[6], hg[7]));
                *reinterpret_cast<uint4*>(dst_u + c0 + v * 8) =
                    make_uint4(pack_bf16x2(hu[0], hu[1]), pack_bf16x2(hu[2], hu[3]), pack_bf16x2(hu[4], hu[5]), pack_bf16x2(hu[6], hu[7]));
                *reinterpret_cast<uint2*>(adst + c0 + v * 8) =
                    make_uint2(cvt_fp8x4<FP8GMM_E4M3>(a[0] * sc, a[1] * sc, a[2] * sc, a[3] * sc),
                               cvt_fp8x4<FP8GMM_E4M3>(a[4] * sc, a[5] * sc, a[6] * sc, a[7] * sc));
              }
            }
          }
        }
        if (p.amax) {
          amax = warp_max(amax);
          if (lane == 0) atomic_max_nonneg(p.amax + t.group * p.amax_stride, amax);
        }
      }
      // hand the accumulator back to the MMA warp (which lives in the leader CTA when paired)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (kCtas == 1) mbar_arrive(tempty_bar(acc)); else mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) bulk_wait_all();  // TMA stores of this warp have been written out
  }

  // ===================== teardown =====================
  tc_fence_before();
  if (kCtas == 2) cluster_sync_all(); else __syncthreads();
  if (*abort_flag) {
    // Give copies and MMAs that are still in flight time to land before shared memory and TMEM go away.
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 200000ull) {
    }
  }
  // A CTA of a pair must not leave while its peer can still touch its shared memory or barriers.
  if (kCtas == 2) cluster_sync_all(); else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (kCtas == 2) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
  }
}

__global__ void __launch_bounds__(kThreads, 1) grouped_gemm_kernel(const __grid_constant__ GemmParams p) { gemm_body<1>(p); }

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    grouped_gemm_pair_kernel(const __grid_constant__ GemmParams p) { gemm_body<2>(p); }

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// 2-D uint8 tensor (rows x cols bytes, row pitch = cols), box 128 rows x 128 bytes, SWIZZLE_128B.
int encode_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols) {
  auto fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return FP8GMM_CUDA_ERROR;
  }
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols};
  const cuuint32_t box[2] = {kBlockK, 128};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with %d (base %p, rows %llu, cols %llu)", static_cast<int>(r), base,
              static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols));
    return FP8GMM_CUDA_ERROR;
  }
  return FP8GMM_OK;
}

// 3-D uint8 tensor (groups x rows x cols bytes), box 1 x 128 rows x 128 bytes, SWIZZLE_128B: the (G, K, N) weights
// read MN-major.  Rows past a group's end are zero-filled (they are out of bounds of the middle dimension), so a
// contraction that is not a multiple of 128 never reads the next group's rows.
int encode_map_3d(CUtensorMap* map, const void* base, uint64_t groups, uint64_t rows, uint64_t cols) {
  auto fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return FP8GMM_CUDA_ERROR;
  }
  const cuuint64_t dims[3] = {cols, rows, groups};
  const cuuint64_t strides[2] = {cols, rows * cols};
  const cuuint32_t box[3] = {kBlockK, 128, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (3-D) failed with %d (base %p, %llu x %llu x %llu)", static_cast<int>(r), base,
              static_cast<unsigned long long>(groups), static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols));
    return FP8GMM_CUDA_ERROR;
  }
  return FP8GMM_OK;
}

// 2-D bf16 tensor (rows x cols, row pitch = cols) for the epilogue's TMA stores: box 32 rows x 64 columns
// (128 bytes per row), SWIZZLE_128B to match the staging layout.
int encode_store_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols) {
  auto fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return FP8GMM_CUDA_ERROR;
  }
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {64, 32};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (store map) failed with %d (base %p, rows %llu, cols %llu)", static_cast<int>(r), base,
              static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols));
    return FP8GMM_CUDA_ERROR;
  }
  return FP8GMM_OK;
}

// Process-wide switches of the GEMM launches.  Defaults come from the environment, read once when the library is
// first used (FP8GMM_GEMM_CTAS=1|2 forces the tile shape, FP8GMM_GEMM_EPILOGUE=direct turns the TMA-store epilogue
// off, FP8GMM_GEMM_NO_TAIL_SPLIT keeps short group tails on pair tiles, FP8GMM_GEMM_SUPER_ROWS=short,long sets the
// super-row heights of the tile order); fp8gmm_set_gemm_variant changes the first three later.
struct Tuning {
  int ctas = 0;             // 0 = choose per call, 1 = single-CTA 128-row tiles, 2 = CTA-pair 256-row tiles
  bool tail_split = true;   // pair tiles: tails of at most 128 rows go to a second launch on 128-row tiles
  bool tma_epilogue = true; // full 32-row slabs leave through shared memory + TMA stores
  int super_rows_short = kSuperRowsShortK;  // rows per super-row of the tile order, contraction <= kLongK
  int super_rows_long = kSuperRowsLongK;    // ... and above (FP8GMM_GEMM_SUPER_ROWS=short,long; multiples of 256)
  bool wave_sync = true;                    // soft wave barrier for long contractions (FP8GMM_GEMM_WAVE_SYNC=0 turns it off)
};
Tuning& tuning() {
  static Tuning t = [] {
    Tuning v;
    const char* e = getenv("FP8GMM_GEMM_CTAS");
    if (e != nullptr) v.ctas = e[0] == '1' ? 1 : e[0] == '2' ? 2 : 0;
    e = getenv("FP8GMM_GEMM_EPILOGUE");
    v.tma_epilogue = !(e != nullptr && e[0] == 'd');
    v.tail_split = getenv("FP8GMM_GEMM_NO_TAIL_SPLIT") == nullptr;
    e = getenv("FP8GMM_GEMM_WAVE_SYNC");
    v.wave_sync = !(e != nullptr && e[0] == '0');
    e = getenv("FP8GMM_GEMM_SUPER_ROWS");
    int a = 0, b = 0;
    if (e != nullptr && sscanf(e, "%d,%d", &a, &b) == 2 && a >= 256 && b >= 256 && a % 256 == 0 && b % 256 == 0) {
      v.super_rows_short = a;
      v.super_rows_long = b;
    }
    return v;
  }();
  return t;
}

uint32_t make_idesc(int a_format, int b_format, int ctas, bool a_mn = false, bool b_mn = false) {
  // tcgen05 instruction descriptor, kind::f8f6f4: [4,6) D format (1 = f32), [7,10) A format, [10,13) B format
  // (0 = e4m3, 1 = e5m2), bits 15/16 = A / B major (0 = K-major, 1 = MN-major), [17,23) N >> 3, [24,29) M >> 4.
  uint32_t d = 0;
  d |= 1u << 4;
  d |= static_cast<uint32_t>(a_format) << 7;
  d |= static_cast<uint32_t>(b_format) << 10;
  d |= static_cast<uint32_t>(kBlockN >> 3) << 17;
  d |= static_cast<uint32_t>((kBlockM * ctas) >> 4) << 24;  // a CTA pair issues M = 256
  if (a_mn) d |= 1u << 15;  // A is MN-major ("transposed") in shared memory
  if (b_mn) d |= 1u << 16;  // B is MN-major
  return d;
}

// Upper bound on the SMs a GEMM launch occupies (fp8gmm_set_gemm_sm_limit; 0 = all).  A persistent grid that
// fills every SM is delayed as a whole when another kernel (an NCCL exchange on a second stream) holds a few SMs.
int g_sm_limit = 0;

// Wave counters of the long-contraction launches: a small ring of words in device memory, one per launch in flight.
constexpr int kWaveSlots = 64;
__device__ unsigned int g_wave_counters[kWaveSlots];
unsigned int* g_wave_addr[64] = {nullptr};
std::mutex g_wave_mutex;
unsigned int g_wave_next = 0;

// Zeroes the next counter on `s` and returns its device address (NULL if the symbol cannot be resolved: no barrier).
unsigned int* next_wave_counter(cudaStream_t s) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  unsigned int* base;
  unsigned int slot;
  {
    std::lock_guard<std::mutex> lock(g_wave_mutex);
    if (g_wave_addr[dev] == nullptr) {
      void* ptr = nullptr;
      if (cudaGetSymbolAddress(&ptr, g_wave_counters) != cudaSuccess) return nullptr;
      g_wave_addr[dev] = static_cast<unsigned int*>(ptr);
    }
    base = g_wave_addr[dev];
    slot = g_wave_next++ % kWaveSlots;
  }
  if (cudaMemsetAsync(base + slot, 0, sizeof(unsigned int), s) != cudaSuccess) return nullptr;
  return base + slot;
}

int launch(GemmParams& p, int ctas, cudaStream_t s) {
  // The attribute is per device and the call is idempotent and cheap, so it is simply repeated.
  int sms = sm_count();
  if (g_sm_limit > 0 && g_sm_limit < sms) sms = g_sm_limit;
  const int workers = sms / ctas > 0 ? sms / ctas : 1;
  const int grid = ctas * (p.total_tiles < workers ? p.total_tiles : workers);
  p.wait_ns = gemm_wait_limit_ns();
  p.wave_counter = (p.mode == kModeRows && p.k > kLongK && tuning().wave_sync && p.total_tiles > workers) ? next_wave_counter(s) : nullptr;
  if (ctas == 2) {
    FP8GMM_CHECK_CUDA(cudaFuncSetAttribute(grouped_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<2>::kSmemBytes));
    grouped_gemm_pair_kernel<<<grid, kThreads, Cfg<2>::kSmemBytes, s>>>(p);
  } else {
    FP8GMM_CHECK_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<1>::kSmemBytes));
    grouped_gemm_kernel<<<grid, kThreads, Cfg<1>::kSmemBytes, s>>>(p);
  }
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return FP8GMM_OK;
}

bool fmt_ok(int f) { return f == FP8GMM_E4M3 || f == FP8GMM_E5M2; }

// ---------------------------------------------------------------------------------------------
// Weight gradients: one host routine behind the three entry points
// ---------------------------------------------------------------------------------------------
enum WgradForm {
  kWgradTransposed,  // operands are the padded-transposed blocks (features x L_g), K-major for the MMA
  kWgradRowMajor     // operands are row slices of the row-major activations (L_g x features), MN-major for the MMA
};

// Validates the arguments, encodes one pair of tensor maps per group into `host_maps` (2 * num_groups entries of
// host memory owned by the caller), copies them to `device_maps` on `s` and launches the kernel.  The copy reads
// `host_maps` from ordinary host memory that the caller releases right after this returns, which a captured graph
// would replay from a dead buffer: the call is refused while `s` is being captured.
int wgrad_launch(const fp8gmm_wgrad_args* a, cudaStream_t s, const char* name, WgradForm form, CUtensorMap* device_maps,
                 CUtensorMap* host_maps) {
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  FP8GMM_CHECK_CUDA(cudaStreamIsCapturing(s, &capture));
  if (capture != cudaStreamCaptureStatusNone) {
    set_error("%s: the stream is being captured; this call stages its per-group descriptors with a copy from temporary "
              "host memory and cannot be part of a CUDA graph", name);
    return FP8GMM_UNSUPPORTED;
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  int ctas = tuning().ctas;
  if (ctas == 0) ctas = a->n >= 256 ? 2 : 1;
  const int64_t tiles_m = (a->n + kBlockM * ctas - 1) / (kBlockM * ctas);
  const int64_t tiles_n = (a->k + kBlockN - 1) / kBlockN;
  FP8GMM_CHECK_ARG(tiles_m * tiles_n * a->num_groups <= INT32_MAX / 2, "%s: problem too large", name);
  memset(host_maps, 0, sizeof(CUtensorMap) * 2 * static_cast<size_t>(a->num_groups));
  p.tile_start[0] = 0;
  for (int g = 0; g < a->num_groups; ++g) {
    const int64_t o0 = a->t_offsets[g], o1 = a->t_offsets[g + 1];
    const int64_t len = o1 - o0;
    FP8GMM_CHECK_ARG(len >= 0 && o1 <= INT32_MAX - 1024, "%s: group %d has a negative or oversized range", name, g);
    FP8GMM_CHECK_ARG(form == kWgradRowMajor || len % 16 == 0,
                     "%s: group %d contraction length %lld must be a multiple of 16", name, g, (long long)len);
    p.row_start[g] = static_cast<int>(o0);
    p.row_start[g + 1] = static_cast<int>(o1);
    p.tile_start[g + 1] = p.tile_start[g] + static_cast<int>(tiles_m * tiles_n);
    if (len > 0) {
      FP8GMM_CHECK_ARG(a->a_t && a->b_t, "%s: NULL operand pointer", name);
      const char* base_a = static_cast<const char*>(a->a_t) + o0 * a->n;
      const char* base_b = static_cast<const char*>(a->b_t) + o0 * a->k;
      // transposed: (features x len) bytes; row-major: (len x features) bytes -- the box is 128 x 128 bytes either way
      const bool t = form == kWgradTransposed;
      int rc = encode_map(&host_maps[2 * g], base_a, static_cast<uint64_t>(t ? a->n : len), static_cast<uint64_t>(t ? len : a->n));
      if (rc != FP8GMM_OK) return rc;
      rc = encode_map(&host_maps[2 * g + 1], base_b, static_cast<uint64_t>(t ? a->k : len), static_cast<uint64_t>(t ? len : a->k));
      if (rc != FP8GMM_OK) return rc;
    }
  }
  // Every descriptor slot this launch reads is rewritten (empty groups get zeroed slots that are never used).  The
  // source is pageable, so the runtime has staged the bytes by the time the call returns.
  FP8GMM_CHECK_CUDA(cudaMemcpyAsync(device_maps, host_maps, sizeof(CUtensorMap) * 2 * static_cast<size_t>(a->num_groups),
                                    cudaMemcpyHostToDevice, s));
  p.maps = device_maps;
  p.c = static_cast<uint16_t*>(a->c);
  p.sa = a->a_scale_inv;
  p.sb = a->b_scale_inv;
  p.sa_stride = a->a_scale_inv_stride;
  p.sb_stride = a->b_scale_inv_stride;
  p.ldc = a->k;
  p.status = device_status_word();
  FP8GMM_CHECK_ARG(p.status != nullptr, "%s: cannot resolve the device status word", name);
  p.mode = kModeWgrad;
  p.mn_major = form == kWgradRowMajor ? 1 : 0;
  p.activation = FP8GMM_ACT_NONE;
  p.num_groups = a->num_groups;
  p.n = static_cast<int>(a->k);
  p.m_fixed = static_cast<int>(a->n);
  p.k = 0;
  p.tiles_n = static_cast<int>(tiles_n);
  p.total_tiles = p.tile_start[a->num_groups];
  p.idesc = make_idesc(a->a_format, a->b_format, ctas, form == kWgradRowMajor, form == kWgradRowMajor);
  p.super_tiles = tuning().super_rows_short / (kBlockM * ctas);
  if (tuning().tma_epilogue) {
    const int rc = encode_store_map(&p.map_c, a->c, static_cast<uint64_t>(a->num_groups) * a->n, static_cast<uint64_t>(a->k));
    if (rc != FP8GMM_OK) return rc;
    p.tma_store = 1;
  }
  return launch(p, ctas, s);
}

// Argument checks shared by the three entry points; *empty is set when there is nothing to do.
int wgrad_check(const fp8gmm_wgrad_args* a, const char* name, int max_groups, bool* empty) {
  *empty = false;
  FP8GMM_CHECK_ARG(a != nullptr, "%s: NULL arguments", name);
  FP8GMM_CHECK_ARG(a->num_groups >= 0 && a->num_groups <= max_groups, "%s: num_groups %d outside [0, %d]", name,
                   a->num_groups, max_groups);
  FP8GMM_CHECK_ARG(fmt_ok(a->a_format) && fmt_ok(a->b_format), "%s: bad fp8 format", name);
  FP8GMM_CHECK_ARG(a->n > 0 && a->k > 0 && a->n % 16 == 0 && a->k % 16 == 0,
                   "%s: N (%lld) and K (%lld) must be positive multiples of 16", name, (long long)a->n, (long long)a->k);
  if (a->num_groups == 0) {
    *empty = true;
    return FP8GMM_OK;
  }
  FP8GMM_CHECK_ARG(a->t_offsets != nullptr && a->c != nullptr, "%s: NULL pointer", name);
  FP8GMM_CHECK_ARG(a->a_scale_inv && a->b_scale_inv, "%s: NULL scale_inv pointer", name);
  FP8GMM_CHECK_ARG((reinterpret_cast<uintptr_t>(a->a_t) | reinterpret_cast<uintptr_t>(a->b_t) |
                    reinterpret_cast<uintptr_t>(a->c)) % 16 == 0, "%s: operand pointers must be 16-byte aligned", name);
  return FP8GMM_OK;
}

int wgrad_with_workspace(const fp8gmm_wgrad_args* a, void* stream, const char* name, WgradForm form) {
  bool empty = false;
  int rc = wgrad_check(a, name, kMaxGroups, &empty);
  if (rc != FP8GMM_OK || empty) return rc;
  FP8GMM_CHECK_ARG(a->workspace != nullptr && a->workspace_bytes >= fp8gmm_wgrad_workspace_bytes(a->num_groups),
                   "%s: workspace of %zu bytes is smaller than the %zu required", name, a->workspace_bytes,
                   fp8gmm_wgrad_workspace_bytes(a->num_groups));
  FP8GMM_CHECK_ARG(reinterpret_cast<uintptr_t>(a->workspace) % 128 == 0, "%s: workspace must be 128-byte aligned", name);
  std::vector<CUtensorMap> maps(static_cast<size_t>(a->num_groups) * 2);
  return wgrad_launch(a, static_cast<cudaStream_t>(stream), name, form, static_cast<CUtensorMap*>(a->workspace), maps.data());
}

}  // namespace
}  // namespace fp8gmm

extern "C" {

int fp8gmm_grouped_gemm(const fp8gmm_gemm_args* a, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(a != nullptr, "grouped_gemm: NULL arguments");
  FP8GMM_CHECK_ARG(a->num_groups >= 0 && a->num_groups <= kMaxGroups, "grouped_gemm: num_groups %d outside [0, %d]",
                   a->num_groups, kMaxGroups);
  FP8GMM_CHECK_ARG(fmt_ok(a->a_format) && fmt_ok(a->b_format), "grouped_gemm: bad fp8 format");
  FP8GMM_CHECK_ARG(a->n > 0 && a->k > 0 && a->n % 16 == 0 && a->k % 16 == 0,
                   "grouped_gemm: N (%lld) and K (%lld) must be positive multiples of 16", (long long)a->n, (long long)a->k);
  FP8GMM_CHECK_ARG(a->activation >= 0 && a->activation <= 3, "grouped_gemm: bad activation %d", a->activation);
  if (a->num_groups == 0) return FP8GMM_OK;
  FP8GMM_CHECK_ARG(a->m_sizes != nullptr, "grouped_gemm: NULL m_sizes");
  FP8GMM_CHECK_ARG(a->a_scale_inv && a->b_scale_inv, "grouped_gemm: NULL scale_inv pointer");
  if (a->activation != FP8GMM_ACT_NONE) {
    FP8GMM_CHECK_ARG(a->act_out != nullptr, "grouped_gemm: activation requested without act_out");
    FP8GMM_CHECK_ARG(a->activation != FP8GMM_ACT_SWIGLU || a->n % 32 == 0, "grouped_gemm: SwiGLU needs N %% 32 == 0");
    FP8GMM_CHECK_ARG(a->activation != FP8GMM_ACT_DSWIGLU || (a->aux_in != nullptr && fmt_ok(a->act_out_format) &&
                                                           reinterpret_cast<uintptr_t>(a->aux_in) % 16 == 0),
                     "grouped_gemm: the SwiGLU-backward epilogue needs a 16-byte aligned aux_in and a valid act_out_format");
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int tile_n = a->activation == FP8GMM_ACT_SWIGLU ? kBlockN / 2 : kBlockN;
  const int64_t n_cols = a->activation == FP8GMM_ACT_SWIGLU ? a->n / 2 : a->n;
  const int64_t tiles_n = (n_cols + tile_n - 1) / tile_n;
  // Paired 256-row tiles halve the operand traffic per SM; they pay off unless many groups are so small that
  // rounding their rows up to 256 wastes much more than rounding up to 128.
  int64_t pad128 = 0, pad256 = 0;
  for (int g = 0; g < a->num_groups; ++g) {
    const int64_t m = a->m_sizes[g];
    FP8GMM_CHECK_ARG(m >= 0, "grouped_gemm: m_sizes[%d] is negative", g);
    pad128 += (m + 127) / 128 * 128;
    pad256 += (m + 255) / 256 * 256;
  }
  int ctas = tuning().ctas;
  if (ctas == 0) ctas = (pad256 * 10 <= pad128 * 11) ? 2 : 1;
  const int tile_m = kBlockM * ctas;
  // With paired tiles a group whose last 256-row tile holds at most 128 rows would spend a whole pair tile on them
  // (every n-tile of it): such tails are left to a second launch of the single-CTA kernel, whose 128-row tile fits.
  const bool split_tails = ctas == 2 && tuning().tail_split;
  int tail_start[kMaxGroups], tail_count[kMaxGroups];
  int64_t rows = 0, tiles = 0, tail_tiles = 0;
  p.tile_start[0] = 0;
  for (int g = 0; g < a->num_groups; ++g) {
    const int64_t m = a->m_sizes[g];
    const int64_t rem = m % (2 * kBlockM);
    const int64_t tail = (split_tails && rem > 0 && rem <= kBlockM) ? rem : 0;
    const int64_t main_rows = m - tail;
    p.row_start[g] = static_cast<int>(rows);
    p.row_count[g] = static_cast<int>(main_rows);
    tail_start[g] = static_cast<int>(rows + main_rows);
    tail_count[g] = static_cast<int>(tail);
    rows += m;
    tiles += ((main_rows + tile_m - 1) / tile_m) * tiles_n;
    tail_tiles += (tail > 0 ? 1 : 0) * tiles_n;
    FP8GMM_CHECK_ARG(rows <= INT32_MAX - 1024 && tiles <= INT32_MAX / 2, "grouped_gemm: problem too large");
    p.tile_start[g + 1] = static_cast<int>(tiles);
  }
  p.row_start[a->num_groups] = static_cast<int>(rows);
  if (rows == 0) return FP8GMM_OK;
  FP8GMM_CHECK_ARG(a->a && a->b && (a->c || a->c_peers || a->activation == FP8GMM_ACT_DSWIGLU), "grouped_gemm: NULL operand pointer");
  FP8GMM_CHECK_ARG((reinterpret_cast<uintptr_t>(a->a) | reinterpret_cast<uintptr_t>(a->b) |
                    reinterpret_cast<uintptr_t>(a->c) | reinterpret_cast<uintptr_t>(a->act_out)) % 16 == 0,
                   "grouped_gemm: operand pointers must be 16-byte aligned");
  FP8GMM_CHECK_ARG(static_cast<int64_t>(a->num_groups) * a->n <= INT32_MAX - 1024, "grouped_gemm: G*N too large");
  int rc = encode_map(&p.map_a, a->a, static_cast<uint64_t>(rows), static_cast<uint64_t>(a->k));
  if (rc != FP8GMM_OK) return rc;
  FP8GMM_CHECK_ARG(a->b_layout == 0 || a->b_layout == 1, "grouped_gemm: bad b_layout %d", a->b_layout);
  FP8GMM_CHECK_ARG(a->b_layout == 0 || a->activation == FP8GMM_ACT_NONE || a->activation == FP8GMM_ACT_DSWIGLU,
                   "grouped_gemm: b_layout 1 has no fused forward activation");
  if (a->b_layout == 1)
    rc = encode_map_3d(&p.map_b, a->b, static_cast<uint64_t>(a->num_groups), static_cast<uint64_t>(a->k), static_cast<uint64_t>(a->n));
  else
    rc = encode_map(&p.map_b, a->b, static_cast<uint64_t>(a->num_groups) * a->n, static_cast<uint64_t>(a->k));
  if (rc != FP8GMM_OK) return rc;
  p.b_mn = a->b_layout;
  p.maps = nullptr;
  p.c = static_cast<uint16_t*>(a->c);
  p.act_out = static_cast<uint8_t*>(a->act_out);
  p.aux_in = static_cast<const uint16_t*>(a->aux_in);
  p.act_format = a->activation == FP8GMM_ACT_DSWIGLU ? a->act_out_format : FP8GMM_E4M3;
  FP8GMM_CHECK_ARG(a->c_row_map == nullptr || a->activation == FP8GMM_ACT_NONE,
                   "grouped_gemm: c_row_map is only supported without a fused activation");
  p.row_map = a->c_row_map;
  FP8GMM_CHECK_ARG(a->c_peers == nullptr || a->c_row_map != nullptr, "grouped_gemm: c_peers needs a c_row_map that names the ranks");
  p.c_peers = reinterpret_cast<const unsigned long long*>(a->c_peers);
  p.sa = a->a_scale_inv;
  p.sb = a->b_scale_inv;
  p.sc = a->act_scale;
  p.amax = a->act_amax;
  p.sa_stride = a->a_scale_inv_stride;
  p.sb_stride = a->b_scale_inv_stride;
  p.sc_stride = a->act_scale_stride;
  p.amax_stride = a->act_amax_stride;
  p.ldc = a->n;
  p.ld_act = a->activation == FP8GMM_ACT_DSWIGLU ? 2 * a->n : n_cols;
  p.status = device_status_word();
  FP8GMM_CHECK_ARG(p.status != nullptr, "grouped_gemm: cannot resolve the device status word");
  p.mode = kModeRows;
  p.activation = a->activation;
  p.num_groups = a->num_groups;
  p.n = static_cast<int>(a->n);
  p.m_fixed = 0;
  p.k = static_cast<int>(a->k);
  p.tiles_n = static_cast<int>(tiles_n);
  p.total_tiles = static_cast<int>(tiles);
  p.idesc = make_idesc(a->a_format, a->b_format, ctas, false, a->b_layout == 1);
  p.super_tiles = (a->k > kLongK ? tuning().super_rows_long : tuning().super_rows_short) / tile_m;
  if (a->activation != FP8GMM_ACT_GELU && a->activation != FP8GMM_ACT_DSWIGLU && a->c_peers == nullptr && tuning().tma_epilogue) {
    rc = encode_store_map(&p.map_c, a->c, static_cast<uint64_t>(rows), static_cast<uint64_t>(a->n));
    if (rc != FP8GMM_OK) return rc;
    p.tma_store = 1;
  }
  if (p.total_tiles > 0) {
    rc = launch(p, ctas, static_cast<cudaStream_t>(stream));
    if (rc != FP8GMM_OK) return rc;
  }
  if (tail_tiles > 0) {
    // second launch: the groups' short tails on 128-row tiles (same operands, maps and epilogue)
    int t = 0;
    for (int g = 0; g < a->num_groups; ++g) {
      p.row_start[g] = tail_start[g];
      p.row_count[g] = tail_count[g];
      p.tile_start[g] = t;
      t += (tail_count[g] > 0 ? 1 : 0) * static_cast<int>(tiles_n);
    }
    p.tile_start[a->num_groups] = t;
    p.total_tiles = t;
    p.idesc = make_idesc(a->a_format, a->b_format, 1, false, a->b_layout == 1);
    p.super_tiles = (a->k > kLongK ? tuning().super_rows_long : tuning().super_rows_short) / kBlockM;
    rc = launch(p, 1, static_cast<cudaStream_t>(stream));
    if (rc != FP8GMM_OK) return rc;
  }
  return FP8GMM_OK;
}

int fp8gmm_set_gemm_sm_limit(int sms) {
  fp8gmm::g_sm_limit = sms > 0 ? sms : 0;
  return FP8GMM_OK;
}

int fp8gmm_set_gemm_variant(int ctas, int tail_split, int tma_epilogue) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(ctas >= 0 && ctas <= 2, "set_gemm_variant: ctas must be 0 (automatic), 1 or 2");
  Tuning& t = tuning();
  t.ctas = ctas;
  t.tail_split = tail_split != 0;
  t.tma_epilogue = tma_epilogue != 0;
  return FP8GMM_OK;
}

size_t fp8gmm_wgrad_workspace_bytes(int num_groups) {
  return num_groups > 0 ? static_cast<size_t>(num_groups) * 2 * sizeof(CUtensorMap) : 0;
}

int fp8gmm_grouped_wgrad(const fp8gmm_wgrad_args* a, void* stream) {
  return fp8gmm::wgrad_with_workspace(a, stream, "grouped_wgrad", fp8gmm::kWgradTransposed);
}

// Weight gradients straight from the row-major FP8 activations: C_g (n x k) = dY_g^T X_g with dY_g = rows
// [offsets[g], offsets[g+1]) of a (sum m x n) matrix and X_g the same rows of a (sum m x k) matrix.  Seen from the
// MMA both operands are MN-major (the feature dimension is contiguous, the contraction runs over rows), which
// tcgen05 takes through the major bits of the instruction descriptor -- so no padded-transposed copies of the
// activations are needed at all.  One tensor map per group and operand bounds the group's rows, and TMA zero-fills
// the rows past its end, so group sizes need no padding either.
int fp8gmm_grouped_wgrad_rowmajor(const fp8gmm_wgrad_args* a, void* stream) {
  return fp8gmm::wgrad_with_workspace(a, stream, "grouped_wgrad_rowmajor", fp8gmm::kWgradRowMajor);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Weight gradient without a caller-provided workspace
// ---------------------------------------------------------------------------------------------
// fp8gmm_grouped_wgrad needs device scratch for its per-group TMA descriptors and takes it from the
// caller.  Some callers have no device memory to give and cannot get any: a training framework that has
// already claimed the whole GPU for its own memory pool (a fresh cudaMalloc then fails, or stalls, because
// cudaMalloc and cudaFree synchronise the device), or a host runtime whose plug-in contract forbids device
// allocation once it is running.  For them the same kernel is offered with its scratch in a fixed array
// that is part of the library image: every GPU that loads the library holds these
// kStaticWgradMaxGroups * 2 * 128 bytes = 32 KiB until the process exits.
//
// What a caller has to know:
//   * at most kStaticWgradMaxGroups (128) groups per call; more is rejected with FP8GMM_UNSUPPORTED;
//   * the call allocates nothing: no cudaMalloc / cudaFree, no allocating library routine, no heap;
//   * the first call on each device looks up the array's device address (the name of a __device__ array is
//     only a host-side handle, not an address a kernel can use) with that device current; make that first
//     call before starting any stream capture.  A call on a stream that is being captured is refused with
//     FP8GMM_UNSUPPORTED (it copies its descriptors from a stack buffer);
//   * all calls on a device share the one array and each call overwrites all of the part it uses, so
//     nothing from an earlier call is ever read; but two calls whose work overlaps on the GPU (different
//     streams, no ordering between them) race on it.  Issue them on one stream or order them yourself;
//   * host threads are serialised inside the call (one lock around encode, copy and launch), so two
//     threads issuing to the same stream cannot interleave their copies and launches.
constexpr int kStaticWgradMaxGroups = 128;
static __device__ __align__(256) unsigned char g_static_wgrad_maps[kStaticWgradMaxGroups * 2 * sizeof(CUtensorMap)];

namespace fp8gmm {
namespace {
CUtensorMap* g_static_wgrad_addr[64] = {nullptr};
std::mutex g_static_wgrad_mutex;

// Device address of g_static_wgrad_maps on the current device, resolved once per device.  The caller holds
// g_static_wgrad_mutex.
int static_wgrad_scratch(CUtensorMap** out) {
  int dev = 0;
  FP8GMM_CHECK_CUDA(cudaGetDevice(&dev));
  FP8GMM_CHECK_ARG(dev >= 0 && dev < 64, "grouped_wgrad_static: device index %d out of range", dev);
  if (g_static_wgrad_addr[dev] == nullptr) {
    void* ptr = nullptr;
    FP8GMM_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_static_wgrad_maps));
    g_static_wgrad_addr[dev] = static_cast<CUtensorMap*>(ptr);
  }
  *out = g_static_wgrad_addr[dev];
  return FP8GMM_OK;
}
}  // namespace
}  // namespace fp8gmm

extern "C" int fp8gmm_grouped_wgrad_static(const fp8gmm_wgrad_args* a, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(a != nullptr, "grouped_wgrad_static: NULL arguments");
  if (a->num_groups > kStaticWgradMaxGroups) {
    set_error("grouped_wgrad_static: %d groups exceed the %d this allocation-free entry point supports; "
              "use fp8gmm_grouped_wgrad with a workspace", a->num_groups, kStaticWgradMaxGroups);
    return FP8GMM_UNSUPPORTED;
  }
  bool empty = false;
  int rc = wgrad_check(a, "grouped_wgrad_static", kStaticWgradMaxGroups, &empty);
  if (rc != FP8GMM_OK || empty) return rc;
  std::lock_guard<std::mutex> lock(g_static_wgrad_mutex);
  CUtensorMap* scratch = nullptr;
  rc = static_wgrad_scratch(&scratch);
  if (rc != FP8GMM_OK) return rc;
  CUtensorMap maps[kStaticWgradMaxGroups * 2];  // host staging on the stack: no heap, no device allocation
  return wgrad_launch(a, static_cast<cudaStream_t>(stream), "grouped_wgrad_static", kWgradTransposed, scratch, maps);
}
