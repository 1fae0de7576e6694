// Multi-tensor pad + cast + transpose kernels (HBM-bound).
//
// One kernel template serves four operations on a list of 2-D tensors:
//   kCast       bf16 (rows x cols) -> fp8 `OType(scale*x)` twice: same shape and padded transpose + amax
//   kDgelu      as kCast on x = in * dgelu_tanh(in2)
//   kDswiglu    SwiGLU backward on in = d(act) (rows x F), in2 = [gate | up] (rows x 2F): two output halves
//   kTranspose  fp8 (rows x cols) -> fp8 padded transpose only
// kCast and kTranspose run in multi_pad_kernel, the two activation-backward modes in act_pad_kernel (same tile
// shape and thread mapping, different register strategy: see there).
// Semantics: reference csrc/multi_pad_fusion.cu:46-153 (transpose), :155-292 (cast), :294-438 (dgelu).
//
// Design for B200: a CTA of 256 threads owns a 128-row x 256-column tile.  Warp w, lane l loads the
// 16 rows [16w, 16w+16) x 8 columns [8l, 8l+8): every warp-level load touches one 512-byte row
// segment (16-byte vectors, fully coalesced), 16 loads are in flight per thread.  Row-major fp8 is
// stored straight from registers (8 bytes per thread, 256 contiguous bytes per warp).  For the
// transposed copy each thread packs, per column, its 16 row values into one 16-byte vector, parks it
// in shared memory ([column][16-byte row chunk], XOR-swizzled so that both the column-wise writes and
// the row-wise reads are bank-conflict free) and the CTA then writes 128 contiguous bytes per column
// (8 lanes x 16 bytes), i.e. full 128-byte lines whenever padded_rows is a multiple of 16.  Ragged
// shapes (cols % 8, unaligned bases, padded_rows % 16) take predicated scalar accesses in the same
// kernel; there is no second "unaligned" launch.  The kernel is latency bound unless enough loads are in
// flight (ncu: long-scoreboard was the top stall at 51 % of DRAM peak when the compiler interleaved loads and
// use), so all 16 row loads of a thread are issued before the first use.  (A variant that staged input tiles
// with cp.async.bulk row copies was measured slower -- 128 small bulk copies per tile cost more than they hide
// -- and taller tiles, 256 or 512 rows, were slower too.)  The tensor table travels in the parameter block
// (no cap on the number of tensors per call: the host splits long lists into launches of kMaxTensors).
#include <cstdlib>
#include <vector>

#include "common.cuh"

namespace fp8gmm {
namespace {

#ifndef FP8GMM_PAD_WARPS
#define FP8GMM_PAD_WARPS 8
#endif
constexpr int kWarps = FP8GMM_PAD_WARPS;  // each warp owns 16 rows of the tile
constexpr int kThreads = 32 * kWarps;
constexpr int kTileRows = 16 * kWarps;
constexpr int kChunks = kTileRows / 16;   // 16-byte row chunks per transposed column
constexpr int kTileCols = 256;
constexpr int kMaxTensors = 256;

enum Mode { kCast = 0, kDgelu = 1, kDswiglu = 2, kTranspose = 3 };

struct PadDesc {
  const void* in;
  const void* in2;
  uint8_t* out;
  uint8_t* out_t;
  const float* scale;
  float* amax;
  int rows;
  int cols;         // tile space; kDswiglu: F (outputs are 2F wide)
  int padded_rows;  // rows of tile space to cover (>= rows when out_t != NULL, else == rows)
  int tiles_n;
  int fast_io;  // 16-byte input loads and 8-byte row-major stores are legal for every tile
  int fast_t;   // 16-byte transposed stores are legal for every tile
  int pad0, pad1;
};

struct PadArgs {
  int num;
  int tile_start[kMaxTensors + 1];
  PadDesc d[kMaxTensors];
};

__device__ __forceinline__ float dgelu_tanh(float x) {
  const float t = tanhf(0.79788456f * x * (1.f + 0.044715f * x * x));
  return 0.5f * x * ((1.f - t * t) * (0.79788456f + 0.1070322243f * x * x)) + 0.5f * (1.f + t);
}

// Insert byte `b` (already in bits 0-7) at byte position `pos` (compile-time after unrolling).
__device__ __forceinline__ uint32_t put_byte(uint32_t word, uint32_t b, int pos) { return word | (b << (8 * pos)); }

template <int kMode, int kFormat>
// Three CTAs per SM for both modes.  (The fp8 -> fp8 transpose fits in 64 registers, but four CTAs per SM measured
// 4.4 TB/s against 5.3 TB/s with three: more CTAs scatter the 128-byte transposed stores over more DRAM pages at once.)
__global__ void __launch_bounds__(kThreads, 3) multi_pad_kernel(const __grid_constant__ PadArgs args) {
  static_assert(kMode == kCast || kMode == kTranspose, "the activation-backward modes use act_pad_kernel");
  constexpr int kHalves = 1;
  extern __shared__ __align__(16) uint8_t smem_t[];  // [col][kTileRows bytes of rows], 16-byte chunks XOR-swizzled
  __shared__ float staging[kThreads / 32];

  const int tile = blockIdx.x;
  const int t = upper_slot(args.tile_start, args.num, tile);
  const PadDesc& d = args.d[t];
  const int local = tile - args.tile_start[t];
  // column tiles fastest (a banded, rows-fastest order that lets consecutive CTAs write consecutive pieces of the same
  // transposed columns was measured: no gain for the transposes, 2 % slower for the cast)
  const int tile_row = (local / d.tiles_n) * kTileRows;
  const int tile_col = (local % d.tiles_n) * kTileCols;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rows = d.rows, cols = d.cols;
  const int64_t ld_in = cols;                                   // row pitch of `in`
  const int64_t ld_io = cols;                                   // row pitch of `out`
  const float scale = (kMode == kTranspose) ? 1.f : (d.scale ? *d.scale : 1.0f);
  const int col0 = tile_col + lane * 8;
  const int row0 = tile_row + warp * 16;
  const bool fast_io = d.fast_io != 0;

  uint32_t tq[kHalves][8][4];  // per half, per column: 16 row bytes
#pragma unroll
  for (int h = 0; h < kHalves; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int w = 0; w < 4; ++w) tq[h][j][w] = 0;
  float amax = 0.f;

  // ---- phase 1: load, convert, row-major store, pack the transposed bytes in registers --------
  if (kMode == kTranspose) {
    const uint8_t* in = static_cast<const uint8_t*>(d.in);
    // all 16 row loads are issued before the first use, so 16 x 8 bytes per thread are in flight
    uint2 pre[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      pre[i] = make_uint2(0, 0);
      if (fast_io && row0 + i < rows && col0 < cols) pre[i] = ld_stream8(in + (int64_t)(row0 + i) * ld_in + col0);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int row = row0 + i;
      uint32_t lo = 0, hi = 0;
      if (row < rows && col0 < cols) {
        const uint8_t* p = in + (int64_t)row * ld_in + col0;
        if (fast_io) {
          lo = pre[i].x;
          hi = pre[i].y;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (col0 + j < cols) {
              const uint32_t b = p[j];
              if (j < 4) lo |= b << (8 * j); else hi |= b << (8 * (j - 4));
            }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t b = ((j < 4 ? lo : hi) >> (8 * (j & 3))) & 0xFFu;
        tq[0][j][i >> 2] = put_byte(tq[0][j][i >> 2], b, i & 3);
      }
    }
  } else {
    const uint16_t* in = static_cast<const uint16_t*>(d.in);
    // all 16 row loads of `in` are issued before the first use: 256 bytes per thread in flight
    uint4 pre[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      pre[i] = make_uint4(0, 0, 0, 0);
      if (fast_io && row0 + i < rows && col0 < cols) pre[i] = ld_stream16(in + (int64_t)(row0 + i) * ld_in + col0);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int row = row0 + i;
      float x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = 0.f;
      const bool live = row < rows && col0 < cols;
      if (live) {
        if (fast_io) {
          const uint4 v = pre[i];
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) x[2 * j] = bf16_lo(w[j]), x[2 * j + 1] = bf16_hi(w[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (col0 + j < cols) {
              x[j] = __uint_as_float((uint32_t)in[(int64_t)row * ld_in + col0 + j] << 16);
            }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(fabsf(x[j]), amax);
      const float* v0 = x;
      const float* v1 = x;
#pragma unroll
      for (int h = 0; h < kHalves; ++h) {
        const float* v = h == 0 ? v0 : v1;
        const uint32_t q01 = cvt_fp8x2<kFormat>(scale * v[0], scale * v[1]);
        const uint32_t q23 = cvt_fp8x2<kFormat>(scale * v[2], scale * v[3]);
        const uint32_t q45 = cvt_fp8x2<kFormat>(scale * v[4], scale * v[5]);
        const uint32_t q67 = cvt_fp8x2<kFormat>(scale * v[6], scale * v[7]);
        const uint32_t lo = q01 | (q23 << 16), hi = q45 | (q67 << 16);
        if (d.out != nullptr && live) {
          uint8_t* p = d.out + (int64_t)row * ld_io + (int64_t)h * cols + col0;
          if (fast_io) {
            st_stream8(p, make_uint2(lo, hi));
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (col0 + j < cols) p[j] = (uint8_t)(((j < 4 ? lo : hi) >> (8 * (j & 3))) & 0xFFu);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t b = ((j < 4 ? lo : hi) >> (8 * (j & 3))) & 0xFFu;
          tq[h][j][i >> 2] = put_byte(tq[h][j][i >> 2], b, i & 3);
        }
      }
    }
  }

  // ---- phase 2/3: transposed copy through shared memory ---------------------------------------
  if (d.out_t != nullptr) {
    const int padded_rows = d.padded_rows;
#pragma unroll
    for (int h = 0; h < kHalves; ++h) {
      if (h > 0) __syncthreads();
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = lane * 8 + j;
        *reinterpret_cast<uint4*>(smem_t + c * kTileRows + ((warp ^ (lane & 7)) << 4)) =
            make_uint4(tq[h][j][0], tq[h][j][1], tq[h][j][2], tq[h][j][3]);
      }
      __syncthreads();
      uint8_t* out_t = d.out_t + (int64_t)h * cols * padded_rows;
      if (d.fast_t) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int idx = it * kThreads + tid;
          const int c = idx / kChunks, chunk = idx % kChunks;
          const int col = tile_col + c, row = tile_row + chunk * 16;
          if (col < cols && row < padded_rows) {
            const uint4 v = *reinterpret_cast<const uint4*>(smem_t + c * kTileRows + ((chunk ^ ((c >> 3) & 7)) << 4));
            st_stream16(out_t + (int64_t)col * padded_rows + row, v);
          }
        }
      } else {
        for (int idx = tid; idx < kTileCols * kTileRows; idx += kThreads) {
          const int c = idx / kTileRows, r = idx % kTileRows;
          const int col = tile_col + c, row = tile_row + r;
          if (col < cols && row < padded_rows)
            out_t[(int64_t)col * padded_rows + row] =
                smem_t[c * kTileRows + (((r >> 4) ^ ((c >> 3) & 7)) << 4) + (r & 15)];
        }
      }
    }
  }

  // ---- amax: one atomic per CTA ------------------------------------------------------------------
  if (kMode != kTranspose && d.amax != nullptr) {
    amax = warp_max(amax);
    if (lane == 0) staging[warp] = amax;
    __syncthreads();
    if (tid < 32) {
      float m = tid < kThreads / 32 ? staging[tid] : 0.f;
      m = warp_max(m);
      if (tid == 0) atomic_max_nonneg(d.amax, m);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Activation-backward variants (kDgelu, kDswiglu): two or three input streams per output.
// Holding 16 rows of every stream plus the packed transposed bytes in registers (as the cast kernel does for
// its single stream) leaves room for one CTA per SM only and too few loads in flight.  Here a thread walks
// its 16 rows in four batches of four: the loads of a batch (4 rows x 2-3 streams x 16 bytes) are issued
// together, the transposed bytes of a batch are one 32-bit word per column and go to shared memory at once.
// About 100 registers, two CTAs per SM.  Shared-memory layout per half: [column][128 row bytes]; inside a
// column the eight 16-byte chunks are XOR-swizzled with the writer's lane & 7 (as in the cast kernel) and the
// four words of a chunk with lane >> 3, which makes the 32-bit stores of a warp hit 32 different banks.
// ---------------------------------------------------------------------------------------------
// kWithT = false is the form without a transposed copy (what the modules launch by default, since the weight-gradient
// GEMM reads the row-major FP8 rows): no shared-memory tile, no byte packing, three CTAs per SM.
template <int kMode, int kFormat, bool kWithT>
__global__ void __launch_bounds__(kThreads, kWithT ? 2 : 3) act_pad_kernel(const __grid_constant__ PadArgs args) {
  static_assert(kWarps == 8, "the word swizzle below assumes 8 warps (128-row tiles)");
  constexpr int kHalves = (kMode == kDswiglu) ? 2 : 1;
  constexpr int kHalfBytes = kTileCols * kTileRows;
  extern __shared__ __align__(16) uint8_t smem_t[];
  __shared__ float staging[kThreads / 32];

  const int tile = blockIdx.x;
  const int t = upper_slot(args.tile_start, args.num, tile);
  const PadDesc& d = args.d[t];
  const int local = tile - args.tile_start[t];
  const int tile_row = (local / d.tiles_n) * kTileRows;
  const int tile_col = (local % d.tiles_n) * kTileCols;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rows = d.rows, cols = d.cols;
  const int64_t ld_in = cols;
  const int64_t ld_io = (kMode == kDswiglu) ? 2 * (int64_t)cols : cols;
  const float scale = d.scale ? *d.scale : 1.0f;
  const int col0 = tile_col + lane * 8;
  const int row0 = tile_row + warp * 16;
  const bool fast_io = d.fast_io != 0;
  const uint16_t* in = static_cast<const uint16_t*>(d.in);
  const uint16_t* in2 = static_cast<const uint16_t*>(d.in2);
  float amax = 0.f;

#pragma unroll 1
  for (int b = 0; b < 4; ++b) {
    uint4 px[4], pg[4], pu[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = row0 + 4 * b + r;
      px[r] = pg[r] = pu[r] = make_uint4(0, 0, 0, 0);
      if (fast_io && row < rows && col0 < cols) {
        px[r] = ld_stream16(in + (int64_t)row * ld_in + col0);
        pg[r] = ld_stream16(in2 + (int64_t)row * ld_io + col0);
        if (kMode == kDswiglu) pu[r] = ld_stream16(in2 + (int64_t)row * ld_io + cols + col0);
      }
    }
    uint32_t tw[kHalves][8];
#pragma unroll
    for (int h = 0; h < kHalves; ++h)
#pragma unroll
      for (int j = 0; j < 8; ++j) tw[h][j] = 0;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = row0 + 4 * b + r;
      const bool live = row < rows && col0 < cols;
      float x[8], y[8], z[8];
      if (fast_io) {
        const uint32_t xw[4] = {px[r].x, px[r].y, px[r].z, px[r].w};
        const uint32_t gw[4] = {pg[r].x, pg[r].y, pg[r].z, pg[r].w};
        const uint32_t uw[4] = {pu[r].x, pu[r].y, pu[r].z, pu[r].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          x[2 * j] = bf16_lo(xw[j]), x[2 * j + 1] = bf16_hi(xw[j]);
          y[2 * j] = bf16_lo(gw[j]), y[2 * j + 1] = bf16_hi(gw[j]);
          z[2 * j] = bf16_lo(uw[j]), z[2 * j + 1] = bf16_hi(uw[j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          x[j] = y[j] = z[j] = 0.f;
          if (live && col0 + j < cols) {
            x[j] = __uint_as_float((uint32_t)in[(int64_t)row * ld_in + col0 + j] << 16);
            y[j] = __uint_as_float((uint32_t)in2[(int64_t)row * ld_io + col0 + j] << 16);
            if (kMode == kDswiglu) z[j] = __uint_as_float((uint32_t)in2[(int64_t)row * ld_io + cols + col0 + j] << 16);
          }
        }
      }
      float v0[8], v1[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (kMode == kDgelu) {
          v0[j] = x[j] * dgelu_tanh(y[j]);
          v1[j] = 0.f;
        } else {  // d gate = dy * up * d silu(gate), d up = dy * silu(gate)
          const float sg = 1.f / (1.f + __expf(-y[j]));
          v0[j] = x[j] * z[j] * (sg * (1.f + y[j] * (1.f - sg)));
          v1[j] = x[j] * (y[j] * sg);
        }
        amax = fmaxf(fabsf(v0[j]), amax);
        if (kMode == kDswiglu) amax = fmaxf(fabsf(v1[j]), amax);
      }
#pragma unroll
      for (int h = 0; h < kHalves; ++h) {
        const float* v = h == 0 ? v0 : v1;
        const uint32_t q01 = cvt_fp8x2<kFormat>(scale * v[0], scale * v[1]);
        const uint32_t q23 = cvt_fp8x2<kFormat>(scale * v[2], scale * v[3]);
        const uint32_t q45 = cvt_fp8x2<kFormat>(scale * v[4], scale * v[5]);
        const uint32_t q67 = cvt_fp8x2<kFormat>(scale * v[6], scale * v[7]);
        const uint32_t lo = q01 | (q23 << 16), hi = q45 | (q67 << 16);
        if (d.out != nullptr && live) {
          uint8_t* p = d.out + (int64_t)row * ld_io + (int64_t)h * cols + col0;
          if (fast_io) {
            st_stream8(p, make_uint2(lo, hi));
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (col0 + j < cols) p[j] = (uint8_t)(((j < 4 ? lo : hi) >> (8 * (j & 3))) & 0xFFu);
          }
        }
        if (kWithT) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t byte = ((j < 4 ? lo : hi) >> (8 * (j & 3))) & 0xFFu;
            tw[h][j] |= byte << (8 * r);
          }
        }
      }
    }
    if (kWithT && d.out_t != nullptr) {
#pragma unroll
      for (int h = 0; h < kHalves; ++h)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = lane * 8 + j;
          *reinterpret_cast<uint32_t*>(smem_t + h * kHalfBytes + c * kTileRows + ((warp ^ (lane & 7)) << 4) +
                                       ((b ^ (lane >> 3)) << 2)) = tw[h][j];
        }
    }
  }

  if (kWithT && d.out_t != nullptr) {
    __syncthreads();
    const int padded_rows = d.padded_rows;
#pragma unroll
    for (int h = 0; h < kHalves; ++h) {
      uint8_t* out_t = d.out_t + (int64_t)h * cols * padded_rows;
      const uint8_t* half = smem_t + h * kHalfBytes;
      if (d.fast_t) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int idx = it * kThreads + tid;
          const int c = idx >> 3, chunk = idx & 7;
          const int col = tile_col + c, row = tile_row + chunk * 16;
          if (col < cols && row < padded_rows) {
            const uint4 v = *reinterpret_cast<const uint4*>(half + c * kTileRows + ((chunk ^ ((c >> 3) & 7)) << 4));
            // the writer of column c was lane c >> 3, so its words sit at position (batch ^ (c >> 6)); c >> 6 == it >> 1
            uint4 o = v;
            if ((it >> 1) & 1) o = make_uint4(o.y, o.x, o.w, o.z);
            if ((it >> 1) & 2) o = make_uint4(o.z, o.w, o.x, o.y);
            st_stream16(out_t + (int64_t)col * padded_rows + row, o);
          }
        }
      } else {
        for (int idx = tid; idx < kTileCols * kTileRows; idx += kThreads) {
          const int c = idx / kTileRows, r = idx % kTileRows;
          const int col = tile_col + c, row = tile_row + r;
          if (col < cols && row < padded_rows)
            out_t[(int64_t)col * padded_rows + row] =
                half[c * kTileRows + (((r >> 4) ^ ((c >> 3) & 7)) << 4) + ((((r >> 2) & 3) ^ (c >> 6)) << 2) + (r & 3)];
        }
      }
    }
  }

  if (d.amax != nullptr) {
    amax = warp_max(amax);
    if (lane == 0) staging[warp] = amax;
    __syncthreads();
    if (tid < 32) {
      float m = tid < kThreads / 32 ? staging[tid] : 0.f;
      m = warp_max(m);
      if (tid == 0) atomic_max_nonneg(d.amax, m);
    }
  }
}

template <int kMode, int kFormat>
int launch_act(const PadArgs& args, cudaStream_t s) {
  bool any_t = false;
  for (int i = 0; i < args.num; ++i) any_t |= args.d[i].out_t != nullptr;
  if (!any_t) {
    act_pad_kernel<kMode, kFormat, false><<<args.tile_start[args.num], kThreads, 0, s>>>(args);
  } else {
    constexpr int kSmem = kTileCols * kTileRows * (kMode == kDswiglu ? 2 : 1);
    if (kSmem > 48 * 1024)
      FP8GMM_CHECK_CUDA(cudaFuncSetAttribute(act_pad_kernel<kMode, kFormat, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    act_pad_kernel<kMode, kFormat, true><<<args.tile_start[args.num], kThreads, kSmem, s>>>(args);
  }
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return FP8GMM_OK;
}

template <int kMode>
int launch_mode(const PadArgs& args, int out_format, cudaStream_t s) {
  const int grid = args.tile_start[args.num];
  constexpr int kSmem = kTileCols * kTileRows;
  if (kMode == kTranspose || out_format == FP8GMM_E4M3) {
    if (kSmem > 48 * 1024)
      FP8GMM_CHECK_CUDA(cudaFuncSetAttribute(multi_pad_kernel<kMode, FP8GMM_E4M3>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    multi_pad_kernel<kMode, FP8GMM_E4M3><<<grid, kThreads, kSmem, s>>>(args);
  } else {
    if (kSmem > 48 * 1024)
      FP8GMM_CHECK_CUDA(cudaFuncSetAttribute(multi_pad_kernel<kMode, FP8GMM_E5M2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    multi_pad_kernel<kMode, FP8GMM_E5M2><<<grid, kThreads, kSmem, s>>>(args);
  }
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return FP8GMM_OK;
}

int flush(PadArgs& args, int mode, int out_format, cudaStream_t s) {
  if (args.num == 0) return FP8GMM_OK;
  int rc = FP8GMM_OK;
  switch (mode) {
    case kCast: rc = launch_mode<kCast>(args, out_format, s); break;
    case kDgelu:
      rc = out_format == FP8GMM_E4M3 ? launch_act<kDgelu, FP8GMM_E4M3>(args, s) : launch_act<kDgelu, FP8GMM_E5M2>(args, s);
      break;
    case kDswiglu:
      rc = out_format == FP8GMM_E4M3 ? launch_act<kDswiglu, FP8GMM_E4M3>(args, s) : launch_act<kDswiglu, FP8GMM_E5M2>(args, s);
      break;
    default: rc = launch_mode<kTranspose>(args, out_format, s); break;
  }
  args.num = 0;
  args.tile_start[0] = 0;
  return rc;
}

int run(const fp8gmm_tensor_desc* descs, int count, int mode, int out_format, void* stream, const char* name) {
  FP8GMM_CHECK_ARG(count >= 0 && (count == 0 || descs != nullptr), "%s: bad descriptor list", name);
  FP8GMM_CHECK_ARG(out_format == FP8GMM_E4M3 || out_format == FP8GMM_E5M2, "%s: bad fp8 format %d", name, out_format);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The tensor table is launched whenever the parameter block is full and once at the end.
  PadArgs direct;
  direct.num = 0;
  direct.tile_start[0] = 0;
  const int in_elem = mode == kTranspose ? 1 : 2;
  for (int i = 0; i < count; ++i) {
    const fp8gmm_tensor_desc& t = descs[i];
    FP8GMM_CHECK_ARG(t.rows >= 0 && t.cols >= 0, "%s: tensor %d has a negative size", name, i);
    FP8GMM_CHECK_ARG(t.rows <= INT32_MAX - 256 && t.cols <= INT32_MAX / 2 - 256, "%s: tensor %d is too large", name, i);
    const int64_t cover_rows = t.out_t ? t.padded_rows : t.rows;
    FP8GMM_CHECK_ARG(!t.out_t || (t.padded_rows >= t.rows && t.padded_rows <= INT32_MAX - 256),
                     "%s: tensor %d: padded_rows %lld < rows %lld", name, i, (long long)t.padded_rows, (long long)t.rows);
    if (cover_rows == 0 || t.cols == 0) continue;
    FP8GMM_CHECK_ARG(t.in != nullptr || t.rows == 0, "%s: tensor %d has a NULL input", name, i);
    FP8GMM_CHECK_ARG(mode == kCast || mode == kTranspose || t.in2 != nullptr || t.rows == 0,
                     "%s: tensor %d has a NULL second input", name, i);
    FP8GMM_CHECK_ARG(mode != kTranspose || t.out_t != nullptr, "%s: tensor %d has a NULL transposed output", name, i);
    const int64_t tiles_m = (cover_rows + kTileRows - 1) / kTileRows;
    const int64_t tiles_n = (t.cols + kTileCols - 1) / kTileCols;
    const int64_t tiles = tiles_m * tiles_n;
    FP8GMM_CHECK_ARG(tiles <= INT32_MAX / 2, "%s: tensor %d is too large", name, i);
    PadDesc p;
    p.in = t.in;
    p.in2 = t.in2;
    p.out = mode == kTranspose ? nullptr : static_cast<uint8_t*>(t.out);
    p.out_t = static_cast<uint8_t*>(t.out_t);
    p.scale = t.scale;
    p.amax = t.amax;
    p.rows = static_cast<int>(t.rows);
    p.cols = static_cast<int>(t.cols);
    p.padded_rows = static_cast<int>(cover_rows);
    p.tiles_n = static_cast<int>(tiles_n);
    const uintptr_t in_bits = reinterpret_cast<uintptr_t>(t.in) | reinterpret_cast<uintptr_t>(t.in2);
    const int in_align = in_elem == 2 ? 16 : 8;
    p.fast_io = (t.cols % 8 == 0) && (in_bits % in_align == 0) && (reinterpret_cast<uintptr_t>(t.out) % 8 == 0);
    p.fast_t = (cover_rows % 16 == 0) && (reinterpret_cast<uintptr_t>(t.out_t) % 16 == 0);
    p.pad0 = p.pad1 = 0;
    PadArgs& dst = direct;
    if (dst.num == kMaxTensors || tiles + dst.tile_start[dst.num] > INT32_MAX) {
      const int rc = flush(dst, mode, out_format, s);
      if (rc != FP8GMM_OK) return rc;
    }
    dst.d[dst.num] = p;
    dst.tile_start[dst.num + 1] = dst.tile_start[dst.num] + static_cast<int>(tiles);
    ++dst.num;
  }
  return flush(direct, mode, out_format, s);
}

}  // namespace
}  // namespace fp8gmm

extern "C" {

int fp8gmm_multi_pad_transpose(const fp8gmm_tensor_desc* descs, int count, void* stream) {
  return fp8gmm::run(descs, count, fp8gmm::kTranspose, FP8GMM_E4M3, stream, "multi_pad_transpose");
}

int fp8gmm_multi_pad_cast_transpose(const fp8gmm_tensor_desc* descs, int count, int out_format, void* stream) {
  return fp8gmm::run(descs, count, fp8gmm::kCast, out_format, stream, "multi_pad_cast_transpose");
}

int fp8gmm_multi_pad_cast_transpose_dgelu(const fp8gmm_tensor_desc* descs, int count, int out_format, void* stream) {
  return fp8gmm::run(descs, count, fp8gmm::kDgelu, out_format, stream, "multi_pad_cast_transpose_dgelu");
}

int fp8gmm_multi_pad_cast_transpose_dswiglu(const fp8gmm_tensor_desc* descs, int count, int out_format, void* stream) {
  return fp8gmm::run(descs, count, fp8gmm::kDswiglu, out_format, stream, "multi_pad_cast_transpose_dswiglu");
}

int fp8gmm_grouped_pad_cast_transpose(const fp8gmm_grouped_cast_args* a, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(a != nullptr && a->num_groups >= 0 && a->cols >= 0, "grouped_pad_cast_transpose: bad arguments");
  FP8GMM_CHECK_ARG(a->num_groups == 0 || a->row_offsets != nullptr, "grouped_pad_cast_transpose: NULL row_offsets");
  FP8GMM_CHECK_ARG(a->out_t == nullptr || a->t_offsets != nullptr, "grouped_pad_cast_transpose: NULL t_offsets");
  FP8GMM_CHECK_ARG(a->activation >= 0 && a->activation <= 2, "grouped_pad_cast_transpose: bad activation");
  const int mode = a->in_is_fp8 ? kTranspose : (a->activation == 1 ? kDgelu : a->activation == 2 ? kDswiglu : kCast);
  const int64_t in_elem = a->in_is_fp8 ? 1 : 2;
  const int64_t out_w = mode == kDswiglu ? 2 * a->cols : a->cols;  // width of out / in2(dswiglu) / out_t rows
  std::vector<fp8gmm_tensor_desc> descs(static_cast<size_t>(a->num_groups));
  for (int g = 0; g < a->num_groups; ++g) {
    fp8gmm_tensor_desc& t = descs[g];
    const int64_t r0 = a->row_offsets[g], r1 = a->row_offsets[g + 1];
    FP8GMM_CHECK_ARG(r1 >= r0, "grouped_pad_cast_transpose: row_offsets must be non-decreasing");
    t.in = static_cast<const char*>(a->in) + r0 * a->cols * in_elem;
    t.in2 = a->in2 ? static_cast<const char*>(a->in2) + r0 * out_w * 2 : nullptr;
    t.out = a->out ? static_cast<char*>(a->out) + r0 * out_w : nullptr;
    t.rows = r1 - r0;
    t.cols = a->cols;
    if (a->out_t) {
      t.out_t = static_cast<char*>(a->out_t) + a->t_offsets[g] * out_w;
      t.padded_rows = a->t_offsets[g + 1] - a->t_offsets[g];
    } else {
      t.out_t = nullptr;
      t.padded_rows = t.rows;
    }
    t.scale = a->scale ? a->scale + g * a->scale_stride : nullptr;
    t.amax = a->amax ? a->amax + g * a->amax_stride : nullptr;
  }
  // without a transposed output the plain cast is the flat quantise kernel's job (same bytes, same amax, no
  // shared-memory staging)
  if (mode == kCast && a->out_t == nullptr) return fp8gmm_multi_quantize(descs.data(), a->num_groups, a->out_format, stream);
  return run(descs.data(), a->num_groups, mode, a->out_format, stream, "grouped_pad_cast_transpose");
}

int fp8gmm_blocked_cast(const fp8gmm_blocked_cast_args* a, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(a != nullptr && a->num_blocks >= 0 && a->cols >= 0, "blocked_cast: bad arguments");
  if (a->num_blocks == 0 || a->cols == 0) return FP8GMM_OK;
  FP8GMM_CHECK_ARG(a->src_start && a->dst_start && a->rows && a->group, "blocked_cast: NULL block array");
  FP8GMM_CHECK_ARG(a->in != nullptr && a->out != nullptr, "blocked_cast: NULL tensor");
  std::vector<fp8gmm_tensor_desc> descs(static_cast<size_t>(a->num_blocks));
  for (int64_t b = 0; b < a->num_blocks; ++b) {
    fp8gmm_tensor_desc& t = descs[b];
    FP8GMM_CHECK_ARG(a->rows[b] >= 0 && a->src_start[b] >= 0 && a->dst_start[b] >= 0 && a->group[b] >= 0,
                     "blocked_cast: block %lld has a negative field", (long long)b);
    t.in = static_cast<const char*>(a->in) + a->src_start[b] * a->cols * 2;
    t.in2 = nullptr;
    t.out = static_cast<char*>(a->out) + a->dst_start[b] * a->cols;
    t.out_t = nullptr;
    t.scale = a->scale ? a->scale + a->group[b] * a->scale_stride : nullptr;
    t.amax = a->amax ? a->amax + a->group[b] * a->amax_stride : nullptr;
    t.rows = a->rows[b];
    t.cols = a->cols;
    t.padded_rows = a->rows[b];
  }
  FP8GMM_CHECK_ARG(a->num_blocks <= INT32_MAX, "blocked_cast: too many blocks");
  return run(descs.data(), static_cast<int>(a->num_blocks), kCast, a->out_format, stream, "blocked_cast");
}

}  // extern "C"
