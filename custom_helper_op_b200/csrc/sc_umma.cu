// Manifold 3-D convolution as an implicit GEMM on the 5th-generation tensor cores (tcgen05), for the
// case the depth-band networks actually run: 3x3x3 filter, stride 1, dilation 1, bfloat16 storage,
// float32 accumulation, 16 or 32 channels.
//
//   D[m][n] = sum_k A[m][k] * B[n][k]     m: 128 output voxels of a tile (one per thread)
//                                          n: output channels (16 / 32)
//                                          k: tap * CIN + input channel  (27 taps)
// A is never materialised in global memory: every thread gathers, for its voxel and each tap, the CIN
// contiguous bf16 channels of the neighbour voxel - resolving the per-pixel depth shift
// d + base_plane[out] - base_plane[nbr] (custom_helper_op/cc/kernels/
// sparse_conv3d_fast_fixed_param_op_gpu.cu.cc:78-113), padding with default_value - and writes them into
// shared memory in the tensor core's canonical K-major layout (8-row x 16-byte core matrices, no
// swizzle).  The filter (27*CIN*COUT bf16) is laid out once per CTA in the same form.  One elected thread
// issues tcgen05.mma (M=128, N=COUT, K=16) per tap and 16 input channels, accumulating in tensor memory;
// tcgen05.commit signals an mbarrier; the four warps then read their 32 accumulator rows back with
// tcgen05.ld, round to bf16 and store 2*COUT contiguous bytes per voxel.
//
// A tile is processed in three rounds of nine taps (one filter row each) so that the A staging buffer is
// 9*128*CIN*2 bytes and several CTAs fit on an SM: while one CTA waits for its MMAs another gathers.
// The image gradient is the same kernel run over out_grad with the filter flipped in all three
// dimensions, channels swapped and zero padding (sparse_conv3d_fast_op.cc:298-323).
//
// Every wait on the mbarrier is bounded; if it ever gives up the kernel raises a device-side flag
// (readable through sc_umma_timeouts()), stops issuing work, frees its tensor memory and returns.
#include <cuda_bf16.h>

#include <atomic>
#include <mutex>

#include "sc_common.cuh"
#include "sc_entry.h"
#include "smem_grant.h"

namespace chop {
namespace {

__device__ int g_umma_timeouts = 0;
// Host-visible mirror of the counter: a mapped, pinned int that sc_umma_watch() publishes to the device on request.
// A kernel that gives up a wait also bumps it, so a host can notice without synchronising with the device.
__device__ int* g_umma_host_mirror = nullptr;
__device__ __forceinline__ void note_timeout() {
  atomicAdd(&g_umma_timeouts, 1);
  int* h = g_umma_host_mirror;
  if (h) {
    atomicAdd_system(h, 1);
    __threadfence_system();
  }
}
__global__ void note_timeout_kernel() { note_timeout(); }
std::atomic<int> g_umma_rows{1};   // tuning knob "umma_rows": 0 = always the per-tap gather

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory matrix descriptor, K-major, no swizzle: start address, leading byte offset (distance
// between core matrices adjacent in K), stride byte offset (distance between 8-row groups), version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// The descriptor of the same layout `bytes` further on (the start-address field counts 16-byte units and a CTA's
// shared memory cannot carry out of it).  Issuing an MMA then costs one addition per operand instead of
// rebuilding the descriptor; a single thread issues them all, so this is the critical path of a tile.
__device__ __forceinline__ uint64_t umma_desc_advance(uint64_t desc, uint32_t bytes) { return desc + (uint64_t)(bytes >> 4); }

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
  uint32_t ok = 0;
  for (int it = 0; it < (1 << 24) && !ok; ++it) {
    asm volatile(
        "{\n.reg .pred P1;\nmbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\nselp.u32 %0, 1, 0, P1;\n}\n"
        : "=r"(ok)
        : "r"(mbar), "r"(parity)
        : "memory");
  }
  return ok != 0;
}

template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t* r);
template <>
__device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                 "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld<32>(uint32_t taddr, uint32_t* r) {
  tmem_ld<16>(taddr, r);
  tmem_ld<16>(taddr + 16, r + 16);
}

// ---- tap geometry (3x3x3, dilation 1, any strides) -------------------------------------------------------
// TG = false, "forward form": the tile's voxels are OUTPUT voxels of the (strided) convolution, grid
//   [B,oH,oW,oD]; a tap reads the input grid [B,H,W,D] (sc_tap in sc_common.cuh).
// TG = true, "transposed form": the tile's voxels are voxels of the fine grid [B,H,W,D]; a tap reads the
//   coarse grid [B,oH,oW,oD] and exists only where row, column and absolute depth are multiples of the
//   strides (sc_tap_t).  At stride 1 the two forms coincide.
struct VoxPos {
  int b, r, c;      // batch, row and column in the fine grid (forward form: of the voxel's centre tap)
  int depth_abs;    // absolute fine depth plane of the voxel
};

// SM (stride mode): 0 = any strides (runtime divisions), 1 = all strides are 1 (no divisions in the gather),
// 2 = all strides are powers of two (the transposed form tests and divides with masks and shifts; it performs
// about a hundred such operations per voxel, which otherwise dominate the kernel).
__device__ __forceinline__ int div_pow2_trunc(int t, int l) { return t >= 0 ? (t >> l) : -((-t) >> l); }

template <bool TG, int SM>
__device__ __forceinline__ VoxPos vox_pos(const ScArgs& a, long long v) {
  VoxPos p;
  constexpr bool S1 = SM == 1;
  const int d1 = (TG || S1) ? a.D : a.oD, d2 = (TG || S1) ? a.W : a.oW, d3 = (TG || S1) ? a.H : a.oH;
  int dz, cc, rr;
  if (v <= 0x7fffffffLL) {   // 64-bit divisions cost several times the rest of this function
    unsigned u = (unsigned)v;
    dz = (int)(u % (unsigned)d1); u /= (unsigned)d1;
    cc = (int)(u % (unsigned)d2); u /= (unsigned)d2;
    rr = (int)(u % (unsigned)d3);
    p.b = (int)(u / (unsigned)d3);
  } else {
    dz = (int)(v % d1); v /= d1;
    cc = (int)(v % d2); v /= d2;
    rr = (int)(v % d3);
    p.b = (int)(v / d3);
  }
  p.r = (TG || S1) ? rr : rr * a.sr;
  p.c = (TG || S1) ? cc : cc * a.sc;
  const int bp = __ldg(a.base_plane + (p.b * a.H + p.r) * a.W + p.c);
  p.depth_abs = (TG || S1) ? dz + bp : (dz + (bp + a.sd - 1) / a.sd) * a.sd;
  return p;
}

// One (fr, fc) column of taps: false if the whole column is padding; otherwise base = index of the source
// pixel's first voxel and shift = what to subtract from the tap's absolute depth.
template <bool TG, int SM>
__device__ __forceinline__ bool tap_column(const ScArgs& a, const VoxPos& p, int fr, int fc, long long& base, int& shift) {
  const int orow = p.r - 1 + fr, ocol = p.c - 1 + fc;
  if (oob(orow, a.H) || oob(ocol, a.W)) return false;
  const int bp = __ldg(a.base_plane + (p.b * a.H + orow) * a.W + ocol);
  if (TG && SM == 2) {
    if ((orow & (a.sr - 1)) != 0 || (ocol & (a.sc - 1)) != 0) return false;   // orow, ocol >= 0 here
    base = (((long long)p.b * a.oH + (orow >> a.ls_r)) * a.oW + (ocol >> a.ls_c)) * a.oD;
    shift = div_pow2_trunc(bp + a.sd - 1, a.ls_d);
  } else if (TG && SM == 0) {
    if ((orow % a.sr) != 0 || (ocol % a.sc) != 0) return false;
    base = (((long long)p.b * a.oH + orow / a.sr) * a.oW + ocol / a.sc) * a.oD;
    shift = (bp + a.sd - 1) / a.sd;
  } else {
    base = ((long long)(p.b * a.H + orow) * a.W + ocol) * a.D;
    shift = bp;
  }
  return true;
}

// Source voxel of tap fz in a column, or -1.
template <bool TG, int SM>
__device__ __forceinline__ long long tap_voxel(const ScArgs& a, const VoxPos& p, long long base, int shift, int fz) {
  const int od = p.depth_abs - 1 + fz;
  if (TG && SM == 2) {
    if ((od & (a.sd - 1)) != 0) return -1;           // two's complement: also right for negative od
    const int cd = (od >> a.ls_d) - shift;            // od is a multiple of sd: the shift divides exactly
    return oob(cd, a.oD) ? -1 : base + cd;
  }
  if (TG && SM == 0) {
    if ((od % a.sd) != 0) return -1;
    const int cd = od / a.sd - shift;
    return oob(cd, a.oD) ? -1 : base + cd;
  }
  const int ind = od - shift;
  return oob(ind, a.D) ? -1 : base + ind;
}

// Filter [27][Cin_f][Cout_f] -> canonical K-major B tiles in shared memory, B[n][k] of tap t at sB + t*tap_bytes
// (forward: n = output channel, k = input channel; DGRAD: the flipped tap with the channels swapped, whose rows are
// contiguous in the filter tensor).  One 16-byte chunk (eight k of one n) per thread and step, its loads independent of
// each other: every CTA repeats this, so it must not be a chain of dependent scalar loads.
template <int CIN, int COUT, bool DGRAD>
__device__ __forceinline__ void stage_filter_tiles(const unsigned short* flt, unsigned char* sB, int tid, uint32_t lbo,
                                                   uint32_t sbo, int tap_bytes) {
  constexpr int KC = CIN / 8;
#pragma unroll 2
  for (int e = tid; e < 27 * COUT * KC; e += 128) {
    const int kg = e % KC, n = (e / KC) % COUT, t = e / (KC * COUT);
    uint4 w;
    if (DGRAD) {
      w = __ldg(reinterpret_cast<const uint4*>(flt + ((size_t)(26 - t) * COUT + n) * CIN + kg * 8));  // f[flip t][ci = n][oc = k]
    } else {
      unsigned h[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) h[i] = __ldg(flt + ((size_t)t * CIN + kg * 8 + i) * COUT + n);        // f[t][ci = k][oc = n]
      w = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
    }
    *reinterpret_cast<uint4*>(sB + t * tap_bytes + (n / 8) * sbo + kg * lbo + (n % 8) * 16) = w;
  }
}

// CIN: channels of the gathered tensor (K per tap), COUT: channels produced (N).
template <int CIN, int COUT, bool DGRAD, int SM>
__global__ void __launch_bounds__(128) sc_umma_kernel(const ScArgs a, const long long nvox, const int ntiles) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t mbar_s;
  __shared__ uint32_t tmem_base_s;
  constexpr int KC = CIN / 8;                     // 16-byte k-chunks per tap
  constexpr uint32_t LBO = 128, SBO = KC * 128;   // core-matrix strides in K and in M/N
  constexpr int A_TAP_BYTES = 128 * CIN * 2;
  constexpr int B_TAP_BYTES = COUT * CIN * 2;
  unsigned char* sB = smem;                       // 27 taps
  unsigned char* sA = smem + 27 * B_TAP_BYTES;    // 9 taps (one filter row)
  const int tid = threadIdx.x, warp = tid >> 5;

  const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(DGRAD ? a.out_grad : a.images);
  __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(DGRAD ? a.images_grad : a.output);

  // ---- filter -> canonical K-major B tiles: B[n][k] of tap t at sB + t*B_TAP_BYTES -----------------------
  {
    stage_filter_tiles<CIN, COUT, DGRAD>(static_cast<const unsigned short*>(a.filters), sB, tid, LBO, SBO, B_TAP_BYTES);
  }
  if (warp == 0) {
    uint32_t slot = smem_u32(&tmem_base_s), ncols = 32;
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&mbar_s)), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;
  const uint32_t mbar = smem_u32(&mbar_s);
  // instruction descriptor: D f32, A/B bf16, both K-major, N = COUT, M = 128
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(COUT >> 3) << 17) | ((128u >> 4) << 24);

  // padding value of the gathered tensor, replicated over 8 bf16 (zero for gradients with respect to images)
  uint4 padv = make_uint4(0, 0, 0, 0);
  if (!a.pad_zero) {
    const unsigned d16 = __ldg(static_cast<const unsigned short*>(a.default_value));
    const unsigned d32 = d16 | (d16 << 16);
    padv = make_uint4(d32, d32, d32, d32);
  }

  uint32_t phase = 0;
  bool alive = true;
  for (int tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x) {
    const long long v = (long long)tile * 128 + tid;
    const bool vvalid = v < nvox;
    VoxPos pos = {0, 0, 0, 0};
    if (vvalid) pos = vox_pos<DGRAD, SM>(a, v);
    unsigned char* a_row = sA + (tid / 8) * SBO + (tid % 8) * 16;

    for (int fr = 0; fr < 3; ++fr) {
      // ---- gather nine taps (filter row fr) into the staging buffer ---------------------------------------
#pragma unroll
      for (int fc = 0; fc < 3; ++fc) {
        long long base = 0;
        int shift = 0;
        const bool inb = vvalid && tap_column<DGRAD, SM>(a, pos, fr, fc, base, shift);
#pragma unroll
        for (int fz = 0; fz < 3; ++fz) {
          const long long sv = inb ? tap_voxel<DGRAD, SM>(a, pos, base, shift, fz) : -1;
          const bool ok = sv >= 0;
          const uint4* p = reinterpret_cast<const uint4*>(src + (size_t)(ok ? sv : 0) * CIN);
          unsigned char* dstA = a_row + (fc * 3 + fz) * A_TAP_BYTES;
#pragma unroll
          for (int kc = 0; kc < KC; ++kc) {
            uint4 x = vvalid ? padv : make_uint4(0, 0, 0, 0);
            if (ok) x = __ldg(p + kc);
            *reinterpret_cast<uint4*>(dstA + kc * LBO) = x;
          }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncthreads();
      // ---- one thread issues the round's MMAs ----------------------------------------------------------------
      if (tid == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int tt = 0; tt < 9; ++tt) {
#pragma unroll
          for (int k16 = 0; k16 < CIN / 16; ++k16) {
            const uint64_t da = umma_desc(smem_u32(sA + tt * A_TAP_BYTES + k16 * 2 * LBO), LBO, SBO);
            const uint64_t db = umma_desc(smem_u32(sB + (fr * 9 + tt) * B_TAP_BYTES + k16 * 2 * LBO), LBO, SBO);
            umma_bf16(tmem, da, db, IDESC, (fr | tt | k16) != 0 ? 1u : 0u);
          }
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
      }
      // ---- everyone waits until the tensor core has consumed the staging buffer ------------------------------
      // one warp polls the mbarrier (every poll is a shared-memory access); the others wait at the hardware barrier
      bool done = true;
      if (warp == 0) done = mbar_wait(mbar, phase);
      phase ^= 1;
      if (!__syncthreads_and(done)) {
        if (tid == 0) note_timeout();
        alive = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    if (!alive) break;

    // ---- epilogue: accumulator rows -> bf16 -> global ------------------------------------------------------------
    uint32_t acc[COUT];
    tmem_ld<COUT>(tmem + ((uint32_t)(warp * 32) << 16), acc);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if (vvalid) {
      uint4* o = reinterpret_cast<uint4*>(dst + (size_t)v * COUT);
#pragma unroll
      for (int q = 0; q < COUT / 8; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(acc[q * 8 + 2 * i]), __uint_as_float(acc[q * 8 + 2 * i + 1]));
          w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        o[q] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    uint32_t ncols = 32;
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ncols) : "memory");
  }
}


// ---- per-tile table of filter columns for the shifted-row kernels -------------------------------------------
// Entry (pixel q of the tile, filter column col) = {first voxel of the neighbour pixel (-1: outside the image,
// -2: the tile has no such pixel), base_plane[pixel] - base_plane[neighbour]}.  The D + 2 rows of a pixel share
// these nine entries, so the CTA computes each once (one entry per thread) instead of once per row.
constexpr int ROWS_TAB = 42 * 9;   // a tile has at most 128 / 3 pixels
__device__ __forceinline__ void rows_tab_write(const ScArgs& a, int2* tab, int tile, int ntiles, int PT, long long npix, int tid) {
  for (int e = tid; e < PT * 9; e += 128) {
    const int q = e / 9, col = e - q * 9;
    const long long pix = (long long)tile * PT + q;
    int2 ent = make_int2(-2, 0);
    if (tile < ntiles && pix < npix) {
      const unsigned p32 = (unsigned)pix;   // pixel counts are validated to fit 31 bits
      const int c = (int)(p32 % (unsigned)a.W);
      const unsigned t = p32 / (unsigned)a.W;
      const int r = (int)(t % (unsigned)a.H), b = (int)(t / (unsigned)a.H);
      const int orow = r - 1 + col / 3, ocol = c - 1 + col % 3;
      ent.x = -1;
      if (!oob(orow, a.H) && !oob(ocol, a.W)) {
        const int np = (b * a.H + orow) * a.W + ocol;
        ent.x = np * a.D;                   // voxel indices fit 31 bits (checked on the host)
        ent.y = __ldg(a.base_plane + pix) - __ldg(a.base_plane + np);
      }
    }
    tab[e] = ent;
  }
}
// Source voxel of row j of pixel q in each column: >= 0, -1 = padding (default_value), -2 = not part of the tile.
__device__ __forceinline__ void rows_tab_read(const int2* tab, int q, int j, int D, bool row_used, int* sv) {
#pragma unroll
  for (int col = 0; col < 9; ++col) {
    int v = -2;
    if (row_used) {
      const int2 e = tab[q * 9 + col];
      const int plane = j - 1 + e.y;
      v = e.x >= 0 ? (oob(plane, D) ? -1 : e.x + plane) : e.x;
    }
    sv[col] = v;
  }
}

// ---------------------------------------------------------------------------------------------------------
// Stride-1 variant with ONE staged copy per neighbour pixel instead of one per tap.
//
// The three depth taps of a filter column (fr, fc) read the same neighbour pixel at consecutive planes, so
// their A operands are the same rows shifted by one.  With SBO = 128 bytes the canonical K-major layout
// stores row r of a 16-byte K-chunk at r*16 bytes, i.e. rows are linear, and a tap's operand is simply the
// column buffer's address plus fz*16 bytes.  A tile therefore holds PT = 128 / (D + 2) pixels, every pixel
// owning D + 2 rows: row (p, j) of column (fr, fc) holds plane j - 1 + base_plane[p] - base_plane[nbr] of
// the neighbour pixel (default_value outside its band or outside the image), and MMA row m = p*(D+2) + d,
// d < D, is output voxel (p, d); the two remaining rows per pixel produce values that are discarded.
// Against the per-tap gather this stages 9 instead of 27 rows per voxel, issues all 27 taps of a tile
// behind one barrier (one commit, one wait) and reads every neighbour plane once.
// ---------------------------------------------------------------------------------------------------------
template <int CIN, int COUT, bool DGRAD>
__global__ void __launch_bounds__(128, CIN <= 16 ? 4 : 2) sc_umma_rows_kernel(const ScArgs a, const int ntiles, const int PT) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t mbar_s;
  __shared__ uint32_t tmem_base_s;
  __shared__ int2 tab_s[ROWS_TAB];
  constexpr int KC = CIN / 8;
  // rows per column buffer: 128 + the two shifted reads; 132 rows make the K-chunk stride 64 bytes off a multiple
  // of 128, so the KC lanes that store the chunks of one row hit different banks
  constexpr int NRB = 132;
  constexpr uint32_t B_LBO = 128, B_SBO = KC * 128;     // filter tiles: K-chunks adjacent, then 8-row groups
  constexpr uint32_t A_LBO = NRB * 16, A_SBO = 128;     // column buffers: rows linear, K-chunks NRB rows apart
  constexpr int B_TAP_BYTES = COUT * CIN * 2;
  constexpr int COL_BYTES = KC * NRB * 16;
  unsigned char* sB = smem;                             // 27 taps
  unsigned char* sX = smem + 27 * B_TAP_BYTES;          // 9 filter columns
  const int tid = threadIdx.x, warp = tid >> 5;

  const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(DGRAD ? a.out_grad : a.images);
  __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(DGRAD ? a.images_grad : a.output);

  {
    stage_filter_tiles<CIN, COUT, DGRAD>(static_cast<const unsigned short*>(a.filters), sB, tid, B_LBO, B_SBO, B_TAP_BYTES);
    // rows 128..135 of every column buffer are only ever read into discarded output rows; keep them defined
    for (int e = tid; e < 9 * KC * (NRB - 128); e += 128) {
      const int rr = e % (NRB - 128), kc = (e / (NRB - 128)) % KC, col = e / ((NRB - 128) * KC);
      *reinterpret_cast<uint4*>(sX + col * COL_BYTES + kc * A_LBO + (128 + rr) * 16) = make_uint4(0, 0, 0, 0);
    }
  }
  if (warp == 0) {
    uint32_t slot = smem_u32(&tmem_base_s), ncols = 32;
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&mbar_s)), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  rows_tab_write(a, tab_s, blockIdx.x, ntiles, PT, (long long)a.B * a.H * a.W, tid);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;
  const uint32_t mbar = smem_u32(&mbar_s);
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(COUT >> 3) << 17) | ((128u >> 4) << 24);

  uint4 padv = make_uint4(0, 0, 0, 0);
  if (!a.pad_zero) {
    const unsigned d16 = __ldg(static_cast<const unsigned short*>(a.default_value));
    const unsigned d32 = d16 | (d16 << 16);
    padv = make_uint4(d32, d32, d32, d32);
  }

  const int H = a.H, W = a.W, D = a.D, RP = D + 2;
  const long long npix = (long long)a.B * H * W;
  const int p_in_tile = tid / RP, j = tid - p_in_tile * RP;   // this thread's row: pixel of the tile, row of the pixel
  const bool row_used = p_in_tile < PT;
  uint32_t phase = 0;
  bool alive = true;
  // Source voxel of this thread's row in each of the nine filter columns of a tile; -1 = padding (default_value),
  // -2 = the row is not part of the tile (zeros).  Voxel indices fit 31 bits (checked on the host).
  long long pix = 0;
  bool rvalid = false;
  int sv[9];
  auto locate = [&](int tile) {   // from the table that rows_tab_write(tile) left in shared memory
    pix = (long long)tile * PT + p_in_tile;
    rvalid = row_used && tile < ntiles && pix < npix;
    rows_tab_read(tab_s, p_in_tile, j, D, row_used, sv);
  };
  // The KC 16-byte chunks of a row are fetched by KC neighbouring lanes (the row's owner hands its source voxel
  // over by shuffle), so a warp-wide load covers whole rows - contiguous 32*16 bytes where the rows are
  // consecutive planes of one pixel - instead of every other 16 bytes of twice the span: half the L1 wavefronts.
  // Pass i of lane l: row 32*warp + l/KC + i*(32/KC), chunk l%KC.
  uint4 val[9][KC];
  const int lane = tid & 31, chunk = lane % KC, lrow = lane / KC;
  auto request = [&]() {
#pragma unroll
    for (int col = 0; col < 9; ++col) {
#pragma unroll
      for (int i = 0; i < KC; ++i) {
        const int sr = __shfl_sync(0xffffffffu, sv[col], lrow + i * (32 / KC));
        val[col][i] = sr == -2 ? make_uint4(0, 0, 0, 0) : padv;
        if (sr >= 0) val[col][i] = __ldg(reinterpret_cast<const uint4*>(src + (size_t)sr * CIN) + chunk);
      }
    }
  };
  locate(blockIdx.x);
  request();
  __syncthreads();   // everybody has read the first tile's table before the loop writes the next one
  const uint64_t da0 = umma_desc(smem_u32(sX), A_LBO, A_SBO);
  const uint64_t db0 = umma_desc(smem_u32(sB), B_LBO, B_SBO);
  for (int tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x) {
    // ---- stage the nine filter columns: this tile's rows were requested a tile ago and waited in registers
    // while the previous tile's MMAs and epilogue ran (the gather latency is the longest step of a tile) --------
    const long long pix_out = pix;
    const bool rvalid_out = rvalid;
    // the next tile's column table (everybody has read the current one: it was consumed before the barrier that
    // closed the previous tile)
    rows_tab_write(a, tab_s, tile + gridDim.x, ntiles, PT, npix, tid);
#pragma unroll
    for (int col = 0; col < 9; ++col) {
      unsigned char* dx = sX + col * COL_BYTES + chunk * A_LBO + (warp * 32 + lrow) * 16;
#pragma unroll
      for (int i = 0; i < KC; ++i) *reinterpret_cast<uint4*>(dx + i * (32 / KC) * 16) = val[col][i];
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int col = 0; col < 9; ++col) {
#pragma unroll
        for (int fz = 0; fz < 3; ++fz) {
#pragma unroll
          for (int k16 = 0; k16 < CIN / 16; ++k16) {
            const uint64_t da = umma_desc_advance(da0, col * COL_BYTES + k16 * 2 * A_LBO + fz * 16);
            const uint64_t db = umma_desc_advance(db0, (col * 3 + fz) * B_TAP_BYTES + k16 * 2 * B_LBO);
            umma_bf16(tmem, da, db, IDESC, (col | fz | k16) != 0 ? 1u : 0u);
          }
        }
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
    }
    locate(tile + gridDim.x);   // table written before the barrier above; read here, before the barrier below
    request();                  // in flight during this tile's MMAs and epilogue
    // one warp polls the mbarrier (every poll is a shared-memory access); the others wait at the hardware barrier
    bool done = true;
    if (warp == 0) done = mbar_wait(mbar, phase);
    phase ^= 1;
    if (!__syncthreads_and(done)) {
      if (tid == 0) note_timeout();
      alive = false;
      break;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- epilogue: MMA row m = this thread's row; it is output voxel (pixel, j) when j < D -----------------------
    uint32_t acc[COUT];
    tmem_ld<COUT>(tmem + ((uint32_t)(warp * 32) << 16), acc);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if (rvalid_out && j < D) {
      uint4* o = reinterpret_cast<uint4*>(dst + ((size_t)pix_out * D + j) * COUT);
#pragma unroll
      for (int q = 0; q < COUT / 8; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(acc[q * 8 + 2 * i]), __uint_as_float(acc[q * 8 + 2 * i + 1]));
          w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        o[q] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    uint32_t ncols = 32;
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ncols) : "memory");
  }
}


// ---------------------------------------------------------------------------------------------------------
// Filter gradient on the tensor cores:  dW[k][n] = sum over voxels m of A[m][k] * G[m][n]
// (k = tap*CIN + input channel, n = output channel, A = the same gathered tile as in the forward pass,
// G = out_grad).  The reduction runs over voxels, so both operands are used "MN-major": the staging
// buffers hold [8 voxels][8 channels] core matrices, 16 voxels per MMA step, and the M dimension of
// the MMA is a group of 128 consecutive k (128/CIN taps).  ceil(27*CIN/128) such groups each own COUT
// tensor-memory columns, and the accumulators stay in tensor memory across ALL voxel tiles of the CTA;
// they are read once at the end and written as this CTA's partial [27*CIN][COUT] slab, which the same
// fixed-order reduction kernel as the generic path sums over the CTAs.
// d(default_value) (dynamic_default only) is accumulated on the CUDA cores while gathering.
// ---------------------------------------------------------------------------------------------------------
// TG = true is the filter gradient of the TRANSPOSED convolution: the voxels are those of the fine grid, the
// gathered tensor (CIN channels) is the op's coarse input under every tap (default_value where there is
// none) and G (COUT channels) its upstream gradient; the slab is written [tap][coarse ch][fine ch] and the
// reduction kernel moves it to filter_grad[flipped tap][fine ch][coarse ch].
template <int CIN, int COUT, bool TG, int SM>
__global__ void __launch_bounds__(128) sc_umma_wgrad_kernel(const ScArgs a, const long long nvox, const int ntiles) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t mbar_s;
  __shared__ uint32_t tmem_base_s;
  __shared__ float red_s[128];
  constexpr int KC = CIN / 8;            // 16-byte channel chunks per tap
  constexpr int TPR = 128 / CIN;         // taps per round (one 128-row M group)
  constexpr int NT = (27 + TPR - 1) / TPR;
  constexpr int TMEM_COLS = NT * COUT <= 32 ? 32 : (NT * COUT <= 64 ? 64 : (NT * COUT <= 128 ? 128 : 256));
  constexpr uint32_t SBO = 128;                    // between 8-channel groups (M / N direction)
  constexpr uint32_t LBO_A = 16 * 128;             // between 8-voxel groups of the A staging tile
  constexpr uint32_t LBO_G = (COUT / 8) * 128;     // between 8-voxel groups of the G tile
  unsigned char* sA = smem;                        // 16 voxel groups x 2048 B
  unsigned char* sG = smem + 16 * LBO_A;           // 16 voxel groups x LBO_G
  float* wsum = reinterpret_cast<float*>(sG + 16 * LBO_G);  // [27][COUT], dynamic_default only
  const int tid = threadIdx.x, warp = tid >> 5;
  const __nv_bfloat16* img = static_cast<const __nv_bfloat16*>(a.images);
  const __nv_bfloat16* og = static_cast<const __nv_bfloat16*>(a.out_grad);

  const bool dyn = !TG && a.dynamic_default;
  if (dyn) {
    const __nv_bfloat16* flt = static_cast<const __nv_bfloat16*>(a.filters);
    for (int e = tid; e < 27 * COUT; e += 128) {
      const int t = e / COUT, n = e % COUT;
      float s = 0.f;
      for (int ci = 0; ci < CIN; ++ci) s += __bfloat162float(flt[((size_t)t * CIN + ci) * COUT + n]);
      wsum[e] = s;
    }
  }
  if (warp == 0) {
    uint32_t slot = smem_u32(&tmem_base_s), ncols = TMEM_COLS;
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&mbar_s)), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;
  const uint32_t mbar = smem_u32(&mbar_s);
  // D f32, A/B bf16, both operands MN-major (bits 15, 16), N = COUT, M = 128
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(COUT >> 3) << 17) |
                             ((128u >> 4) << 24);
  const unsigned d16 = __ldg(static_cast<const unsigned short*>(a.default_value));
  const unsigned d32 = d16 | (d16 << 16);
  const uint4 padv = make_uint4(d32, d32, d32, d32);
  const uint4 zero4 = make_uint4(0, 0, 0, 0);

  uint32_t phase = 0;
  bool alive = true;
  bool first = true;
  float dacc = 0.f;
  unsigned char* a_row = sA + (tid / 8) * LBO_A + (tid % 8) * 16;
  unsigned char* g_row = sG + (tid / 8) * LBO_G + (tid % 8) * 16;

  for (int tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x) {
    const long long v = (long long)tile * 128 + tid;
    const bool vvalid = v < nvox;
    VoxPos pos = {0, 0, 0, 0};
    float gf[COUT];
#pragma unroll
    for (int n = 0; n < COUT; ++n) gf[n] = 0.f;
    if (vvalid) pos = vox_pos<TG, SM>(a, v);
    // out_grad row of this voxel -> G tile (previous tile's MMAs have completed: every round waits)
#pragma unroll
    for (int nc = 0; nc < COUT / 8; ++nc) {
      uint4 x = zero4;
      if (vvalid) x = __ldg(reinterpret_cast<const uint4*>(og + (size_t)v * COUT) + nc);
      *reinterpret_cast<uint4*>(g_row + nc * SBO) = x;
      if (dyn) {
        const unsigned w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          gf[nc * 8 + 2 * i] = __uint_as_float(w4[i] << 16);
          gf[nc * 8 + 2 * i + 1] = __uint_as_float(w4[i] & 0xffff0000u);
        }
      }
    }

    for (int rd = 0; rd < NT; ++rd) {
      // ---- gather the taps of M group rd ---------------------------------------------------------------------
#pragma unroll
      for (int tt = 0; tt < TPR; ++tt) {
        const int t = rd * TPR + tt;
        bool ok = false;
        bool real_tap = t < 27;
        size_t off = 0;
        if (real_tap && vvalid) {
          const int fz = t % 3, fc = (t / 3) % 3, fr = t / 9;
          long long base = 0;
          int shift = 0;
          if (tap_column<TG, SM>(a, pos, fr, fc, base, shift)) {
            const long long sv = tap_voxel<TG, SM>(a, pos, base, shift, fz);
            if (sv >= 0) {
              ok = true;
              off = (size_t)sv * CIN;
            }
          }
          if (!ok && dyn) {
            // fixed_param_op_gpu.cu.cc:273-277: d(default) += sum_n (sum_ci filter[t][ci][n]) * out_grad[m][n]
            const float* ws = wsum + t * COUT;
#pragma unroll
            for (int n = 0; n < COUT; ++n) dacc = fmaf(ws[n], gf[n], dacc);
          }
        }
#pragma unroll
        for (int kc = 0; kc < KC; ++kc) {
          uint4 x = (real_tap && vvalid) ? padv : zero4;
          if (ok) x = __ldg(reinterpret_cast<const uint4*>(img + off) + kc);
          *reinterpret_cast<uint4*>(a_row + (tt * KC + kc) * SBO) = x;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncthreads();
      if (tid == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // 16 voxels (two 8-voxel groups) per MMA
          const uint64_t da = umma_desc(smem_u32(sA + ks * 2 * LBO_A), LBO_A, SBO);
          const uint64_t db = umma_desc(smem_u32(sG + ks * 2 * LBO_G), LBO_G, SBO);
          umma_bf16(tmem + rd * COUT, da, db, IDESC, (first && ks == 0) ? 0u : 1u);
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
      }
      // one warp polls the mbarrier (every poll is a shared-memory access); the others wait at the hardware barrier
      bool done = true;
      if (warp == 0) done = mbar_wait(mbar, phase);
      phase ^= 1;
      if (!__syncthreads_and(done)) {
        if (tid == 0) note_timeout();
        alive = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    first = false;
  }

  // ---- accumulators -> this CTA's partial slab -----------------------------------------------------------------
  constexpr int K = 27 * CIN;
  float* part = static_cast<float*>(a.workspace) + (size_t)blockIdx.x * ((size_t)K * COUT + 1);
  if (alive) {
#pragma unroll
    for (int rd = 0; rd < NT; ++rd) {
      uint32_t acc[COUT];
      if (!first) {
        tmem_ld<COUT>(tmem + ((uint32_t)(warp * 32) << 16) + rd * COUT, acc);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
      const int k = rd * 128 + tid;
      if (k < K) {
#pragma unroll
        for (int n = 0; n < COUT; ++n) part[(size_t)k * COUT + n] = first ? 0.f : __uint_as_float(acc[n]);
      }
    }
  }
  red_s[tid] = dacc;
  __syncthreads();
  for (int o = 64; o > 0; o >>= 1) {
    if (tid < o) red_s[tid] += red_s[tid + o];
    __syncthreads();
  }
  if (tid == 0) part[(size_t)K * COUT] = red_s[0];

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    uint32_t ncols = TMEM_COLS;
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ncols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------
// Stride-1 filter gradient with the column buffers of sc_umma_rows_kernel (16 gathered channels).
//
// The buffers hold, per 16-byte chunk q = (filter column, channel chunk), the rows of a tile at 16 bytes each -
// which is also the MN-major layout with the voxels as the reduction dimension (LBO = 128: eight voxels per core
// matrix, linear beyond; SBO = the chunk stride).  For a depth tap fz the operand is again the buffer address plus
// fz*16 bytes; out_grad (the other operand) is not shifted and carries zeros in the rows that are not voxels.
// One MMA block of M = 128 covers chunks 0..15 = filter columns 0..7; the ninth column is taken from a second
// block that starts at chunk 2 (columns 1..8, only its last 16 rows are kept) - the tensor pipe is idle anyway
// and no dummy shared memory is needed.  3 depth taps x 2 blocks x COUT tensor-memory columns accumulate over
// all tiles of the CTA.  One barrier per tile instead of four, 9 staged rows per voxel instead of 27.
// TG (transposed convolution) only changes the operand roles, exactly as in sc_umma_wgrad_kernel.
// ---------------------------------------------------------------------------------------------------------
template <int COUT, bool TG>
__global__ void __launch_bounds__(128, 4) sc_umma_wgrad_rows_kernel(const ScArgs a, const int ntiles, const int PT) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t mbar_s;
  __shared__ uint32_t tmem_base_s;
  __shared__ float red_s[128];
  constexpr int CIN = 16, KC = 2;
  constexpr int NRB = 132;                         // as in sc_umma_rows_kernel
  constexpr uint32_t X_SBO = NRB * 16;             // chunk stride (M direction)
  constexpr uint32_t X_LBO = 128;                  // eight voxels further (reduction direction): rows are linear
  // out_grad tile with the three depth taps side by side in N: chunk fz*(COUT/8) + nc of voxel group m'/8 holds
  // channels nc*8.. of out_grad row m' - fz, so ONE MMA with N = 3*COUT per 16 tile rows serves the three taps
  // (an N = 16 MMA costs the issuing thread as much as an N = 48 one, and that thread is the tile's critical path)
  constexpr int NCH = 3 * (COUT / 8);              // 16-byte chunks per row of the widened tile
  constexpr uint32_t G_SBO = 128, G_LBO = NCH * 128;
  constexpr int TMEM_COLS = 6 * COUT <= 128 ? 128 : 256;
  unsigned char* sX = smem;                        // 18 chunks x NRB rows x 16 B
  unsigned char* sG = smem + 18 * X_SBO;           // 16 voxel groups x G_LBO
  float* wsum = reinterpret_cast<float*>(sG + 16 * G_LBO);   // [27][COUT], dynamic_default only
  const int tid = threadIdx.x, warp = tid >> 5;
  const __nv_bfloat16* img = static_cast<const __nv_bfloat16*>(a.images);
  const __nv_bfloat16* og = static_cast<const __nv_bfloat16*>(a.out_grad);

  const bool dyn = !TG && a.dynamic_default;
  if (dyn) {
    const __nv_bfloat16* flt = static_cast<const __nv_bfloat16*>(a.filters);
    for (int e = tid; e < 27 * COUT; e += 128) {
      const int t = e / COUT, n = e % COUT;
      float sum = 0.f;
      for (int ci = 0; ci < CIN; ++ci) sum += __bfloat162float(flt[((size_t)t * CIN + ci) * COUT + n]);
      wsum[e] = sum;
    }
  }
  // rows 0 (tap 1) and 0, 1 (tap 2) of the widened out_grad tile have no source row: zero, once
  if (tid < 3 * (COUT / 8)) {
    const int which = tid / (COUT / 8), nc = tid % (COUT / 8);          // (tap 1,row 0), (tap 2,row 0), (tap 2,row 1)
    const int fz = which == 0 ? 1 : 2, row = which == 2 ? 1 : 0;
    *reinterpret_cast<uint4*>(sG + (fz * (COUT / 8) + nc) * G_SBO + row * 16) = make_uint4(0, 0, 0, 0);
  }
  for (int e = tid; e < 18 * (NRB - 128); e += 128)   // rows 128..135: only multiplied by zero rows of out_grad, but
    *reinterpret_cast<uint4*>(sX + (e / (NRB - 128)) * X_SBO + (128 + e % (NRB - 128)) * 16) = make_uint4(0, 0, 0, 0);  // must be finite
  if (warp == 0) {
    uint32_t slot = smem_u32(&tmem_base_s), ncols = TMEM_COLS;
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&mbar_s)), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;
  const uint32_t mbar = smem_u32(&mbar_s);
  // D f32, A/B bf16, both operands MN-major (bits 15, 16), N = COUT, M = 128
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)((3 * COUT) >> 3) << 17) |
                             ((128u >> 4) << 24);
  const unsigned d16 = __ldg(static_cast<const unsigned short*>(a.default_value));
  const unsigned d32 = d16 | (d16 << 16);
  const uint4 padv = make_uint4(d32, d32, d32, d32);
  const uint4 zero4 = make_uint4(0, 0, 0, 0);

  const int H = a.H, W = a.W, D = a.D, RP = D + 2;
  const long long npix = (long long)a.B * H * W;
  const int p_in_tile = tid / RP, j = tid - p_in_tile * RP;
  const bool row_used = p_in_tile < PT;
  uint32_t phase = 0;
  bool alive = true, first = true;
  float dacc = 0.f;

  // This thread's row of a tile: its pixel, its out_grad row (zeros for rows that are not voxels) and its source
  // voxel (or -1) in each of the nine filter columns (as in sc_umma_rows_kernel).
  bool rvalid = false;
  int sv[9];                                         // -1 = padding, -2 = row not in the tile
  unsigned padmask = 0;                              // bit col: this row of column col is padding
  uint4 gx[COUT / 8];
  auto locate = [&](int tile) {
    const long long pix = (long long)tile * PT + p_in_tile;
    rvalid = row_used && tile < ntiles && pix < npix;
    const bool is_voxel = rvalid && j < D;          // rows j = D, D+1 of a pixel are halo rows, not output voxels
    int b = 0, r = 0, c = 0, bp_out = 0;
    if (rvalid) {
      const unsigned p32 = (unsigned)pix;   // pixel counts are validated to fit 31 bits
      c = (int)(p32 % (unsigned)W);
      const unsigned t = p32 / (unsigned)W;
      r = (int)(t % (unsigned)H);
      b = (int)(t / (unsigned)H);
      bp_out = __ldg(a.base_plane + pix);
    }
#pragma unroll
    for (int nc = 0; nc < COUT / 8; ++nc) {
      gx[nc] = zero4;
      if (is_voxel) gx[nc] = __ldg(reinterpret_cast<const uint4*>(og + ((size_t)pix * D + j) * COUT) + nc);
    }
    padmask = 0;
#pragma unroll
    for (int col = 0; col < 9; ++col) {
      const int orow = r - 1 + col / 3, ocol = c - 1 + col % 3;
      const bool inb = rvalid && !oob(orow, H) && !oob(ocol, W);
      const int np = inb ? (b * H + orow) * W + ocol : 0;
      const int plane = j - 1 + bp_out - __ldg(a.base_plane + np);
      const bool ok = inb && !oob(plane, D);
      sv[col] = ok ? np * D + plane : (rvalid ? -1 : -2);
      if (!ok) padmask |= 1u << col;
    }
  };
  locate(blockIdx.x);
  const uint64_t da0 = umma_desc(smem_u32(sX), X_LBO, X_SBO);
  const uint64_t db0 = umma_desc(smem_u32(sG), G_LBO, G_SBO);

  for (int tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x) {
    // this thread's out_grad row m goes to row m + fz of tap block fz (rows 126, 127 are never voxels)
#pragma unroll
    for (int fz = 0; fz < 3; ++fz) {
      const int m = tid + fz;
      if (m < 128) {
        unsigned char* g_row = sG + (m / 8) * G_LBO + (m % 8) * 16 + fz * (COUT / 8) * G_SBO;
#pragma unroll
        for (int nc = 0; nc < COUT / 8; ++nc) *reinterpret_cast<uint4*>(g_row + nc * G_SBO) = gx[nc];
      }
    }
    const bool rvalid_cur = rvalid;
    const unsigned padmask_cur = padmask;
    // the two 16-byte chunks of a row are fetched by neighbouring lanes (see sc_umma_rows_kernel)
    uint4 val[9][KC];
    const int lane = tid & 31, chunk = lane % KC, lrow = lane / KC;
#pragma unroll
    for (int col = 0; col < 9; ++col) {
#pragma unroll
      for (int i = 0; i < KC; ++i) {
        const int sr = __shfl_sync(0xffffffffu, sv[col], lrow + i * (32 / KC));
        val[col][i] = sr == -2 ? zero4 : padv;
        if (sr >= 0) val[col][i] = __ldg(reinterpret_cast<const uint4*>(img + (size_t)sr * CIN) + chunk);
      }
    }
    locate(tile + gridDim.x);   // the next tile's lookups and out_grad row run while this tile's rows are in flight
#pragma unroll
    for (int col = 0; col < 9; ++col) {
      unsigned char* dx = sX + (col * KC + chunk) * X_SBO + (warp * 32 + lrow) * 16;
#pragma unroll
      for (int i = 0; i < KC; ++i) *reinterpret_cast<uint4*>(dx + i * (32 / KC) * 16) = val[col][i];
    }

    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {   // 16 tile rows (two 8-row groups) per MMA
          const uint64_t da = umma_desc_advance(da0, blk * 2 * X_SBO + ks * 2 * X_LBO);
          const uint64_t db = umma_desc_advance(db0, ks * 2 * G_LBO);
          umma_bf16(tmem + blk * 3 * COUT, da, db, IDESC, (first && ks == 0) ? 0u : 1u);
        }
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
    }
    if (dyn) {
      // fixed_param_op_gpu.cu.cc:273-277: d(default) += sum_n (sum_ci filter[tap][ci][n]) * out_grad[voxel][n] over the
      // padded taps.  This thread's row j of column col is tap (col, fz) of voxel d = j - fz of the same pixel; the
      // G tile (read here, behind the barrier above) holds that voxel's out_grad row at tile row tid - fz.
      for (int fz = 0; fz < 3; ++fz) {
        const int dv = j - fz;
        if (!rvalid_cur || dv < 0 || dv >= D || padmask_cur == 0) continue;
        const unsigned char* grow = sG + ((tid - fz) / 8) * G_LBO + ((tid - fz) % 8) * 16;
        float gf[COUT];
#pragma unroll
        for (int nc = 0; nc < COUT / 8; ++nc) {
          const uint4 x = *reinterpret_cast<const uint4*>(grow + nc * G_SBO);
          const unsigned w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            gf[nc * 8 + 2 * i] = __uint_as_float(w4[i] << 16);
            gf[nc * 8 + 2 * i + 1] = __uint_as_float(w4[i] & 0xffff0000u);
          }
        }
        for (int col = 0; col < 9; ++col) {
          if (!((padmask_cur >> col) & 1u)) continue;
          const float* ws = wsum + (col * 3 + fz) * COUT;
#pragma unroll
          for (int n = 0; n < COUT; ++n) dacc = fmaf(ws[n], gf[n], dacc);
        }
      }
    }
    // one warp polls the mbarrier (every poll is a shared-memory access); the others wait at the hardware barrier
    bool done = true;
    if (warp == 0) done = mbar_wait(mbar, phase);
    phase ^= 1;
    if (!__syncthreads_and(done)) {
      if (tid == 0) note_timeout();
      alive = false;
      break;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    first = false;
  }

  // ---- accumulators -> this CTA's partial slab [27*CIN][COUT] (+ default-value gradient) -------------------
  constexpr int K = 27 * CIN;
  float* part = static_cast<float*>(a.workspace) + (size_t)blockIdx.x * ((size_t)K * COUT + 1);
  if (alive) {
#pragma unroll
    for (int fz = 0; fz < 3; ++fz) {
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        uint32_t acc[COUT];
        if (!first) {
          tmem_ld<COUT>(tmem + ((uint32_t)(warp * 32) << 16) + (blk * 3 + fz) * COUT, acc);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        }
        // MMA row tid of block blk is chunk q = 2*blk + tid/8, element tid%8: column q/2, channel (q%2)*8 + tid%8.
        // Block 0 supplies columns 0..7, block 1 only column 8 (its rows 112..127).
        const int q = 2 * blk + tid / 8;
        const int col = q / KC, ci = (q % KC) * 8 + (tid % 8);
        if (blk == 0 || col == 8) {
          const int k = (col * 3 + fz) * CIN + ci;
#pragma unroll
          for (int n = 0; n < COUT; ++n) part[(size_t)k * COUT + n] = first ? 0.f : __uint_as_float(acc[n]);
        }
      }
    }
  }
  red_s[tid] = dacc;
  __syncthreads();
  for (int o = 64; o > 0; o >>= 1) {
    if (tid < o) red_s[tid] += red_s[tid + o];
    __syncthreads();
  }
  if (tid == 0) part[(size_t)K * COUT] = red_s[0];

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    uint32_t ncols = TMEM_COLS;
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ncols) : "memory");
  }
}

// Sum of element e over the slabs warp, warp + 8, warp + 16, ... in a fixed order, four loads in flight (the
// slabs are 27*CIN*COUT*4 bytes apart, so every load is a separate DRAM/L2 access and one at a time is latency-bound).
__device__ __forceinline__ float slab_column_sum(const float* col, size_t stride, int first, int nparts) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int p = first;
  for (; p + 24 < nparts; p += 32) {
    const float a0 = col[(size_t)p * stride], a1 = col[(size_t)(p + 8) * stride], a2 = col[(size_t)(p + 16) * stride],
                a3 = col[(size_t)(p + 24) * stride];
    s0 += a0; s1 += a1; s2 += a2; s3 += a3;
  }
  for (; p < nparts; p += 8) s0 += col[(size_t)p * stride];
  return (s0 + s1) + (s2 + s3);
}

// Sum of the per-CTA partial slabs in a fixed order (deterministic).  A block owns 32 consecutive
// elements; its 8 warps each add every 8th slab with coalesced 128-byte reads, then the 8 warp sums are
// added in warp order.  Element n_el is the default-value gradient.
__global__ void __launch_bounds__(256) sc_umma_wgrad_reduce(const float* part, int nparts, long long n_el, float* filter_grad,
                                                            float* default_grad) {
  __shared__ float sm[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long e = (long long)blockIdx.x * 32 + lane;
  float s = 0.f;
  if (e <= n_el) s = slab_column_sum(part + e, (size_t)(n_el + 1), warp, nparts);
  sm[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && e <= n_el) {
    float t = sm[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) t += sm[w][lane];
    if (e < n_el) filter_grad[e] = t;
    else *default_grad = t;
  }
}

// Transposed convolution: slab element [tap][kc][n] (kc: coarse channel of KC, n: fine channel of NC) ->
// filter_grad[26 - tap][n][kc]; same fixed summation order.
__global__ void __launch_bounds__(256) sc_umma_wgrad_reduce_t(const float* part, int nparts, int KC, int NC, float* filter_grad) {
  __shared__ float sm[8][32];
  const long long n_el = (long long)27 * KC * NC;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long e = (long long)blockIdx.x * 32 + lane;
  float s = 0.f;
  if (e < n_el) s = slab_column_sum(part + e, (size_t)(n_el + 1), warp, nparts);
  sm[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && e < n_el) {
    float t = sm[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) t += sm[w][lane];
    const int n = (int)(e % NC), kc = (int)((e / NC) % KC), tap = (int)(e / ((long long)NC * KC));
    filter_grad[((long long)(26 - tap) * NC + n) * KC + kc] = t;
  }
}

template <int COUT, bool TG>
int launch_wgrad_rows(const ScArgs& a, int nparts, cudaStream_t st) {
  auto k = sc_umma_wgrad_rows_kernel<COUT, TG>;
  const size_t smem = (size_t)18 * 132 * 16 + (size_t)16 * 3 * (COUT / 8) * 128 + (size_t)27 * COUT * 4 + 1024;
  if (int e = grant_smem(k, smem)) return e;
  const int PT = 128 / (a.D + 2);
  const long long npix = (long long)a.B * a.H * a.W;
  const long long ntiles = (npix + PT - 1) / PT;
  if (nparts > ntiles) nparts = (int)ntiles;
  k<<<nparts, 128, smem, st>>>(a, (int)ntiles, PT);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const long long n_el = (long long)27 * 16 * COUT;
  if (TG)
    sc_umma_wgrad_reduce_t<<<(unsigned)((n_el + 31) / 32), 256, 0, st>>>(static_cast<const float*>(a.workspace), nparts, 16, COUT,
                                                                          static_cast<float*>(a.filter_grad));
  else
    sc_umma_wgrad_reduce<<<(unsigned)((n_el + 1 + 31) / 32), 256, 0, st>>>(static_cast<const float*>(a.workspace), nparts, n_el,
                                                                             static_cast<float*>(a.filter_grad),
                                                                             static_cast<float*>(a.default_grad));
  return (int)cudaGetLastError();
}

template <int CIN, int COUT, bool TG>
int launch_wgrad(const ScArgs& a, int nparts, cudaStream_t st) {
  const bool s1 = a.sr == 1 && a.sc == 1 && a.sd == 1;
  if constexpr (CIN == 16) {
    if (s1 && a.D + 2 <= 128 && g_umma_rows.load()) return launch_wgrad_rows<COUT, TG>(a, nparts, st);
  }
  auto k = s1 ? sc_umma_wgrad_kernel<CIN, COUT, TG, 1>
              : ((TG && a.ls_r >= 0) ? sc_umma_wgrad_kernel<CIN, COUT, TG, TG ? 2 : 0> : sc_umma_wgrad_kernel<CIN, COUT, TG, 0>);
  const size_t smem = (size_t)16 * 2048 + (size_t)16 * (COUT / 8) * 128 + (size_t)27 * COUT * 4 + 1024;
  if (int e = grant_smem(k, smem)) return e;
  const long long nvox = TG ? a.nvox_in : a.nvox_out;
  const int ntiles = (int)((nvox + 127) / 128);
  if (nparts > ntiles) nparts = ntiles;  // a persistent CTA per slab: more CTAs than tiles would leave slabs unwritten
  k<<<nparts, 128, smem, st>>>(a, nvox, ntiles);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const long long n_el = (long long)27 * CIN * COUT;
  if (TG)
    sc_umma_wgrad_reduce_t<<<(unsigned)((n_el + 31) / 32), 256, 0, st>>>(static_cast<const float*>(a.workspace), nparts, CIN,
                                                                          COUT, static_cast<float*>(a.filter_grad));
  else
    sc_umma_wgrad_reduce<<<(unsigned)((n_el + 1 + 31) / 32), 256, 0, st>>>(static_cast<const float*>(a.workspace), nparts, n_el,
                                                                             static_cast<float*>(a.filter_grad),
                                                                             static_cast<float*>(a.default_grad));
  return (int)cudaGetLastError();
}

template <int CIN, int COUT, bool DGRAD>
int launch_rows(const ScArgs& a, cudaStream_t st) {
  auto k = sc_umma_rows_kernel<CIN, COUT, DGRAD>;
  const size_t smem = (size_t)27 * COUT * CIN * 2 + (size_t)9 * (CIN / 8) * 132 * 16 + 1024;
  if (int e = grant_smem(k, smem)) return e;
  const int PT = 128 / (a.D + 2);
  const long long npix = (long long)a.B * a.H * a.W;
  const long long ntiles = (npix + PT - 1) / PT;
  int per_sm = (int)((size_t)220 * 1024 / (smem + 2048));
  if (per_sm > 8) per_sm = 8;
  if (per_sm < 1) per_sm = 1;
  long long grid = 148LL * per_sm;
  if (grid > ntiles) grid = ntiles;
  k<<<(unsigned)grid, 128, smem, st>>>(a, (int)ntiles, PT);
  return (int)cudaGetLastError();
}


template <int CIN, int COUT, bool DGRAD>
int launch(const ScArgs& a, long long nvox, cudaStream_t st) {
  // stride 1 and a band of at most 126 planes: the shifted-row kernel
  if (a.sr == 1 && a.sc == 1 && a.sd == 1 && a.D + 2 <= 128 && g_umma_rows.load()) return launch_rows<CIN, COUT, DGRAD>(a, st);
  const bool s1 = a.sr == 1 && a.sc == 1 && a.sd == 1;
  auto k = s1 ? sc_umma_kernel<CIN, COUT, DGRAD, 1>
              : ((DGRAD && a.ls_r >= 0) ? sc_umma_kernel<CIN, COUT, DGRAD, DGRAD ? 2 : 0> : sc_umma_kernel<CIN, COUT, DGRAD, 0>);
  const size_t smem = (size_t)27 * COUT * CIN * 2 + (size_t)9 * 128 * CIN * 2 + 1024;
  if (int e = grant_smem(k, smem)) return e;
  const int ntiles = (int)((nvox + 127) / 128);
  int per_sm = (int)((size_t)220 * 1024 / (smem + 2048));
  if (per_sm > 8) per_sm = 8;
  if (per_sm < 1) per_sm = 1;
  int grid = 148 * per_sm;
  if (grid > ntiles) grid = ntiles;
  k<<<grid, 128, smem, st>>>(a, nvox, ntiles);
  return (int)cudaGetLastError();
}

}  // namespace

bool sc_umma_supported(int dtype, const ScArgs& a) {
  return dtype == 2 && a.fh == 3 && a.fw == 3 && a.fd == 3 && a.dr == 1 && a.dc == 1 && a.dd == 1 &&
         (a.Cin == 16 || a.Cin == 32) && (a.Cout == 16 || a.Cout == 32) && a.nvox_in < ((long long)1 << 31) - 128;
}

int sc_umma_fwd_launch(const ScArgs& a, cudaStream_t st) {
  if (a.Cin == 16 && a.Cout == 16) return launch<16, 16, false>(a, a.nvox_out, st);
  if (a.Cin == 16 && a.Cout == 32) return launch<16, 32, false>(a, a.nvox_out, st);
  if (a.Cin == 32 && a.Cout == 16) return launch<32, 16, false>(a, a.nvox_out, st);
  return launch<32, 32, false>(a, a.nvox_out, st);
}

// gathers out_grad (Cout channels) and produces images_grad (Cin channels)
int sc_umma_dgrad_launch(const ScArgs& a, cudaStream_t st) {
  if (a.Cin == 16 && a.Cout == 16) return launch<16, 16, true>(a, a.nvox_in, st);
  if (a.Cin == 16 && a.Cout == 32) return launch<32, 16, true>(a, a.nvox_in, st);
  if (a.Cin == 32 && a.Cout == 16) return launch<16, 32, true>(a, a.nvox_in, st);
  return launch<32, 32, true>(a, a.nvox_in, st);
}

// nparts partial slabs of (27*Cin*Cout + 1) floats must fit in the workspace; every CTA writes one.
int sc_umma_wgrad_launch(const ScArgs& a, int nparts, cudaStream_t st) {
  if (a.Cin == 16 && a.Cout == 16) return launch_wgrad<16, 16, false>(a, nparts, st);
  if (a.Cin == 16 && a.Cout == 32) return launch_wgrad<16, 32, false>(a, nparts, st);
  if (a.Cin == 32 && a.Cout == 16) return launch_wgrad<32, 16, false>(a, nparts, st);
  return launch_wgrad<32, 32, false>(a, nparts, st);
}

// Filter gradient of the transposed convolution: gathers a.images (coarse, Cout channels) under the taps of
// every fine voxel, G = a.out_grad (fine, Cin channels).
int sc_umma_twgrad_launch(const ScArgs& a, int nparts, cudaStream_t st) {
  if (a.Cin == 16 && a.Cout == 16) return launch_wgrad<16, 16, true>(a, nparts, st);
  if (a.Cin == 16 && a.Cout == 32) return launch_wgrad<32, 16, true>(a, nparts, st);
  if (a.Cin == 32 && a.Cout == 16) return launch_wgrad<16, 32, true>(a, nparts, st);
  return launch_wgrad<32, 32, true>(a, nparts, st);
}

void sc_umma_set_rows(int on) { g_umma_rows = on; }

int sc_umma_timeouts() {
  int v = -1;
  if (cudaMemcpyFromSymbol(&v, g_umma_timeouts, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

namespace {
std::mutex g_watch_mu;
int* g_watch_host = nullptr;          // mapped pinned int, shared by all devices of the process
unsigned long long g_watch_devs = 0;  // devices that know its address (bit = device ordinal, < 64)
}  // namespace

// Number of abandoned waits seen through the host-visible mirror; -1 if it cannot be set up.  The first call per
// device allocates (once per process) and publishes the mirror - that call synchronises; later calls read host memory.
int sc_umma_watch() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  std::lock_guard<std::mutex> lk(g_watch_mu);
  if (!g_watch_host) {
    int* h = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&h), sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    *h = 0;
    g_watch_host = h;
  }
  if (!((g_watch_devs >> dev) & 1ull)) {
    int* dptr = nullptr;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&dptr), g_watch_host, 0) != cudaSuccess ||
        cudaMemcpyToSymbol(g_umma_host_mirror, &dptr, sizeof(dptr)) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    g_watch_devs |= 1ull << dev;
  }
  return *const_cast<volatile int*>(g_watch_host);
}

// Test facility (behind the tuning opt-in): on != 0 runs the give-up bookkeeping once (default stream), without any wait;
// on == 0 clears the device counter of the current device and the mirror.
int sc_umma_note_timeout_for_test(int on) {
  if (on) {
    note_timeout_kernel<<<1, 1>>>();
    return (int)cudaGetLastError();
  }
  const int zero = 0;
  if (cudaMemcpyToSymbol(g_umma_timeouts, &zero, sizeof(int)) != cudaSuccess) return (int)cudaGetLastError();
  std::lock_guard<std::mutex> lk(g_watch_mu);
  if (g_watch_host) *const_cast<volatile int*>(g_watch_host) = 0;
  return 0;
}

}  // namespace chop
