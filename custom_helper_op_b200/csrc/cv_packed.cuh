// CostVolume (KIND 1, MEAN, fused arithmetic) kernels on packed single-precision pairs.
//
// Same work decomposition as cv_tuned.cuh - a warp owns 32/LG neighbouring pixels, LG = C/4 lanes per
// pixel, four channels per lane; phase A projects one voxel per lane into every view, phase B does the
// channel work with the 2x2 texel footprint cached in registers along the planes - but every per-channel
// quantity lives in a 64-bit register holding two floats from the 16-byte load to the 16-byte store, and
// the arithmetic is issued as fma/mul/add/sub.f32x2 (two channels per instruction).  What phase B needs
// per (plane, view) is laid out by phase A so that no pair ever has to be assembled in the inner loop:
//   rec  {dw, dw, dh, dh}   one 16-byte broadcast shared load gives both splatted interpolation weights
//   chg  one bit per plane  "the footprint differs from the previous plane's" (a ballot of phase A), so
//                           the texel index is read only where the footprint is reloaded
// Accumulators and footprints are updated in place (asm operands tied to their registers), so the compiler has
// nothing to copy where the control flow of the reload joins.
// The projection itself stays unfused and in the reference's order (cv_project.cuh), so the validity
// count is bit-exact; cost meets the float tolerance (same formulas as cv_fwd_tuned).  The gradient stays with
// cv_bwd_tuned: a packed-pair gradient kernel was measured slower (fewer instructions, but the pair arithmetic
// takes two pipe cycles and its records doubled the shared-memory loads).
// Reference: custom_helper_op/cc/kernels/cost_volume_kernels_gpu.cu.cc:33-131.
#pragma once
#include <type_traits>

#include "cv_project.cuh"

namespace chop {

typedef unsigned long long pk2;  // two floats in one 64-bit register: {low, high} = channels {c, c+1}

__device__ __forceinline__ pk2 pk_fma(pk2 a, pk2 b, pk2 c) {
  pk2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ pk2 pk_mul(pk2 a, pk2 b) {
  pk2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ pk2 pk_add(pk2 a, pk2 b) {
  pk2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ pk2 pk_sub(pk2 a, pk2 b) {
  pk2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ pk2 pk_make(float lo, float hi) {
  pk2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void pk_split(pk2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// A lane's four channels as two pairs.
template <typename T>
struct PkLoad;
template <>
struct PkLoad<float> {
  static __device__ __forceinline__ void ld(const float* p, pk2& a, pk2& b) {
    asm("ld.global.nc.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p));
  }
};
template <>
struct PkLoad<__nv_bfloat16> {
  static __device__ __forceinline__ void ld(const __nv_bfloat16* p, pk2& a, pk2& b) {
    const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
    a = pk_make(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u));
    b = pk_make(__uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
  }
};

// 16-byte streaming store of two pairs (the cost volume is written once and not re-read here).
__device__ __forceinline__ void pk_store_stream(float* p, pk2 a, pk2 b) {
  asm volatile("st.global.cs.v2.b64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
// acc += a * b with the accumulator updated in place (the operand is tied to its register)
__device__ __forceinline__ void pk_fma_to(pk2& acc, pk2 a, pk2 b) { asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b)); }

// The cached 2x2 footprint of one view as differences against the reference pixel.  The reload is one asm block
// that updates the eight registers in place; a view that does not see the plane reads the reference pixel four
// times instead (dx = dy = 0), which makes every difference an exact zero: the "empty footprint".
struct Footprint {
  pk2 a0a, a0b, ua, ub, va, vb, ta, tb;  // t00 - ref, t10 - t00, t01 - t00, t11 - t01 - (t10 - t00); channel pairs {0,1}, {2,3}
};

// p: this lane's channels of texel (fh, fw); dx / dy: bytes to the next texel of the row / to the next row.
template <typename T>
struct FootprintLoad;
template <>
struct FootprintLoad<float> {
  static __device__ __forceinline__ void go(Footprint& f, const float* p, long long dx, long long dy, pk2 ref0, pk2 ref1) {
    asm("{\n\t"
        ".reg .b64 q<8>, px, py, pxy;\n\t"
        "add.s64 px, %8, %9;\n\t"
        "add.s64 py, %8, %10;\n\t"
        "add.s64 pxy, py, %9;\n\t"
        "ld.global.nc.v2.b64 {q0, q1}, [%8];\n\t"
        "ld.global.nc.v2.b64 {q2, q3}, [px];\n\t"
        "ld.global.nc.v2.b64 {q4, q5}, [py];\n\t"
        "ld.global.nc.v2.b64 {q6, q7}, [pxy];\n\t"
        "sub.rn.f32x2 %0, q0, %11;\n\t"
        "sub.rn.f32x2 %1, q1, %12;\n\t"
        "sub.rn.f32x2 %2, q4, q0;\n\t"
        "sub.rn.f32x2 %3, q5, q1;\n\t"
        "sub.rn.f32x2 %4, q2, q0;\n\t"
        "sub.rn.f32x2 %5, q3, q1;\n\t"
        "sub.rn.f32x2 %6, q6, q2;\n\t"
        "sub.rn.f32x2 %7, q7, q3;\n\t"
        "sub.rn.f32x2 %6, %6, %2;\n\t"
        "sub.rn.f32x2 %7, %7, %3;\n\t"
        "}"
        : "+l"(f.a0a), "+l"(f.a0b), "+l"(f.ua), "+l"(f.ub), "+l"(f.va), "+l"(f.vb), "+l"(f.ta), "+l"(f.tb)
        : "l"(p), "l"(dx), "l"(dy), "l"(ref0), "l"(ref1));
  }
};
template <>
struct FootprintLoad<__nv_bfloat16> {
  static __device__ __forceinline__ void go(Footprint& f, const __nv_bfloat16* p, long long dx, long long dy, pk2 ref0, pk2 ref1) {
    asm("{\n\t"
        ".reg .b64 q<8>, px, py, pxy;\n\t"
        ".reg .b32 w<8>, lo, hi;\n\t"
        "add.s64 px, %8, %9;\n\t"
        "add.s64 py, %8, %10;\n\t"
        "add.s64 pxy, py, %9;\n\t"
        "ld.global.nc.v2.b32 {w0, w1}, [%8];\n\t"
        "ld.global.nc.v2.b32 {w2, w3}, [px];\n\t"
        "ld.global.nc.v2.b32 {w4, w5}, [py];\n\t"
        "ld.global.nc.v2.b32 {w6, w7}, [pxy];\n\t"
        "shl.b32 lo, w0, 16;\n\t and.b32 hi, w0, 0xffff0000;\n\t mov.b64 q0, {lo, hi};\n\t"
        "shl.b32 lo, w1, 16;\n\t and.b32 hi, w1, 0xffff0000;\n\t mov.b64 q1, {lo, hi};\n\t"
        "shl.b32 lo, w2, 16;\n\t and.b32 hi, w2, 0xffff0000;\n\t mov.b64 q2, {lo, hi};\n\t"
        "shl.b32 lo, w3, 16;\n\t and.b32 hi, w3, 0xffff0000;\n\t mov.b64 q3, {lo, hi};\n\t"
        "shl.b32 lo, w4, 16;\n\t and.b32 hi, w4, 0xffff0000;\n\t mov.b64 q4, {lo, hi};\n\t"
        "shl.b32 lo, w5, 16;\n\t and.b32 hi, w5, 0xffff0000;\n\t mov.b64 q5, {lo, hi};\n\t"
        "shl.b32 lo, w6, 16;\n\t and.b32 hi, w6, 0xffff0000;\n\t mov.b64 q6, {lo, hi};\n\t"
        "shl.b32 lo, w7, 16;\n\t and.b32 hi, w7, 0xffff0000;\n\t mov.b64 q7, {lo, hi};\n\t"
        "sub.rn.f32x2 %0, q0, %11;\n\t"
        "sub.rn.f32x2 %1, q1, %12;\n\t"
        "sub.rn.f32x2 %2, q4, q0;\n\t"
        "sub.rn.f32x2 %3, q5, q1;\n\t"
        "sub.rn.f32x2 %4, q2, q0;\n\t"
        "sub.rn.f32x2 %5, q3, q1;\n\t"
        "sub.rn.f32x2 %6, q6, q2;\n\t"
        "sub.rn.f32x2 %7, q7, q3;\n\t"
        "sub.rn.f32x2 %6, %6, %2;\n\t"
        "sub.rn.f32x2 %7, %7, %3;\n\t"
        "}"
        : "+l"(f.a0a), "+l"(f.a0b), "+l"(f.ua), "+l"(f.ub), "+l"(f.va), "+l"(f.vb), "+l"(f.ta), "+l"(f.tb)
        : "l"(p), "l"(dx), "l"(dy), "l"(ref0), "l"(ref1));
  }
};

// Shared-memory bytes per warp: row products, one 16-byte record and one texel index per (view, lane),
// the splatted 1/views per lane, one change word per view.
__host__ __device__ inline size_t packed_fwd_smem_per_warp(int N, int G) {
  return (size_t)N * G * sizeof(Coef<float>) + (size_t)N * 32 * 16 + 32 * 8 + (size_t)N * 32 * 4 +
         (((size_t)N * 4 + 15) & ~(size_t)15);
}

#ifndef CHOP_PK_FWD_BLOCKS
#define CHOP_PK_FWD_BLOCKS 3
#endif

template <typename T, int C>
__global__ void __launch_bounds__(256, CHOP_PK_FWD_BLOCKS) cv_fwd_packed(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LG = C / 4;
  constexpr int G = 32 / LG;
  static_assert(LG * 4 == C && (LG & (LG - 1)) == 0 && LG >= 2 && LG <= 8, "C in {8, 16, 32}");
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int li = lane & (LG - 1);
  const int g = lane / LG;

  const long long item = (long long)blockIdx.x * warps + wib;
  if (item >= (long long)a.npb * a.nchunks) return;
  const int chunk_id = (int)(item / a.npb);
  const int pb = (int)(item - (long long)chunk_id * a.npb);
  const long long pix0 = (long long)pb * G;
  const bool pvalid = pix0 + g < a.npix;
  const long long pix = pvalid ? pix0 + g : a.npix - 1;
  const int dlo = a.d_begin + chunk_id * a.chunk;
  const int dhi = min(a.d_end, dlo + a.chunk);
  const int N = a.N;
  const int D = a.D;

  unsigned char* mine = smem_raw + (size_t)wib * smem_per_warp;
  Coef<float>* coef = reinterpret_cast<Coef<float>*>(mine);
  float4* rec = reinterpret_cast<float4*>(coef + N * G);   // [N][32] {dw, dw, dh, dh}
  float2* inv2 = reinterpret_cast<float2*>(rec + N * 32);  // [32]    {1/views, 1/views}
  int* tex = reinterpret_cast<int*>(inv2 + 32);            // [N][32] top-left texel or -1
  unsigned* chg = reinterpret_cast<unsigned*>(tex + N * 32);  // [N] bit (g*LG + j): reload at plane j

  stage_coefs<float>(a, coef, lane, G, pix0);
  __syncwarp();

  const T* src_lane = static_cast<const T*>(a.src) + li * 4;
  const T* ref_lane = static_cast<const T*>(a.ref) + pix * C + li * 4;
  pk2 ref0, ref1;
  PkLoad<T>::ld(ref_lane, ref0, ref1);
  const int b = (int)(pix / ((long long)a.H * a.W));
  const float base = static_cast<const float*>(a.depth)[pix];
  const float* offs = static_cast<const float*>(a.offsets) + (long long)b * D;
  const long long dx_bytes = (long long)C * (long long)sizeof(T);
  const long long dy_bytes = (long long)a.Ws * dx_bytes;
  float* out = static_cast<float*>(a.cost) + (pix * D + dlo) * C + li * 4;
  const ulonglong2* rec_mine = reinterpret_cast<const ulonglong2*>(rec) + g * LG;
  const int* tex_mine = tex + g * LG;
  const pk2* inv_mine = reinterpret_cast<const pk2*>(inv2) + g * LG;

  for (int dblk = dlo; dblk < dhi; dblk += LG, out += LG * C) {
    // ---- phase A: lane (g, li) projects plane dblk+li of pixel g into every view ---------------------
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      const float depth = dv ? xadd(base, offs[d]) : 0.0f;
      int used = 0;
      for (int n = 0; n < N; ++n) {
        int t = -1;
        float dh = 0.0f, dw = 0.0f;
        if (dv) {
          float gh, gw;
          t = project<float, false>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, dh, dw, gh, gw);
          used += t >= 0;
        }
        rec[n * 32 + lane] = make_float4(dw, dw, dh, dh);
        tex[n * 32 + lane] = t;
        // the footprint registers do not outlive a (block, view): plane 0 always loads
        const int prev = __shfl_up_sync(0xffffffffu, t, 1);
        const unsigned bal = __ballot_sync(0xffffffffu, li == 0 || t != prev);
        if (lane == 0) chg[n] = bal;
      }
      if (dv) __stcs(a.mask + pix * D + d, used);
      const float inv = used > 0 ? 1.0f / (float)used : 0.0f;
      inv2[lane] = make_float2(inv, inv);
    }
    __syncwarp();

    // ---- phase B ---------------------------------------------------------------------------------------
    if (pvalid) {
      pk2 acc[LG][2];
#pragma unroll
      for (int j = 0; j < LG; ++j) acc[j][0] = acc[j][1] = 0ull;
      for (int n = 0; n < N; ++n) {
        const ulonglong2* r = rec_mine + n * 32;
        const int* tx = tex_mine + n * 32;
        const unsigned m = chg[n] >> (g * LG);
        Footprint F;
        F.a0a = F.a0b = F.ua = F.ub = F.va = F.vb = F.ta = F.tb = 0ull;
#pragma unroll
        for (int j = 0; j < LG; ++j) {
          if (j == 0 || ((m >> j) & 1u)) {   // the footprint registers do not outlive a (block, view): plane 0 always loads
            const int t = tx[j];
            const T* p = t >= 0 ? src_lane + (size_t)t * C : ref_lane;
            FootprintLoad<T>::go(F, p, t >= 0 ? dx_bytes : 0ll, t >= 0 ? dy_bytes : 0ll, ref0, ref1);
          }
          const ulonglong2 wh = r[j];  // x = {dw, dw}, y = {dh, dh}
          const pk2 X0 = pk_fma(F.ta, wh.x, F.ua);
          const pk2 X1 = pk_fma(F.tb, wh.x, F.ub);
          const pk2 Y0 = pk_fma(wh.x, F.va, F.a0a);
          const pk2 Y1 = pk_fma(wh.x, F.vb, F.a0b);
          const pk2 d0 = pk_fma(wh.y, X0, Y0);  // sample - ref
          const pk2 d1 = pk_fma(wh.y, X1, Y1);
          pk_fma_to(acc[j][0], d0, d0);
          pk_fma_to(acc[j][1], d1, d1);
        }
      }

      const int left = dhi - dblk;
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        if (j < left) {
          const pk2 inv = inv_mine[j];
          pk_store_stream(out + j * C, pk_mul(acc[j][0], inv), pk_mul(acc[j][1], inv));
        }
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------------------
// forward, plane-major nest, for a compile-time number of source views NV <= 2
//
// With few views the footprints of ALL views fit in registers (16 per view), so the nest can be
//     depth block -> plane -> view
// instead of block -> view -> plane: a plane's cost is finished and stored before the next plane
// starts (no accumulator array: 28 fewer registers), and a view's footprint survives from one block of
// planes to the next - it is reloaded only where the texel really changes, not at every block start.
// The kernel is bound by the time one warp needs for its chain of dependent steps (measured: the same binary
// runs 2.3x faster with three resident CTAs per SM than with one, while extra arithmetic, shared loads or an
// L2-resident output change nothing), so it keeps the chain short and the per-lane loads low:
//   * the row products of the pixel (Coef) stay in registers for the whole work item;
//   * the division by the view count needs no load: with at most two views it is a multiplication by
//     one half where both see the voxel (a ballot bit), by one otherwise (zero views give an exact zero);
//   * the reload is one asm block that updates the eight footprint registers in place; a view that does
//     not see the plane reads the reference pixel four times instead, which makes all differences zero.
// ---------------------------------------------------------------------------------------------------
// project<> without branches: every operation is executed (a non-positive z only produces values that the
// validity test then discards), so the independent chains of several views can be interleaved by the
// compiler.  Same unfused operations in the same order as project<float,false>: identical results.
__device__ __forceinline__ int project_nb(const Coef<float>& c, float depth, int half_centor, int Hs, int Ws, float& dh, float& dw) {
  const float z = xadd(xmul(c.zc, depth), c.t2);
  const float w3 = xadd(xmul(c.wc, depth), c.t0);
  const float h3 = xadd(xmul(c.hc, depth), c.t1);
  float sw = xdiv(w3, z);
  float sh = xdiv(h3, z);
  if (half_centor) {
    sw = xsub(sw, 0.5f);
    sh = xsub(sh, 0.5f);
  }
  const bool ok = (z > 0.0f) & (sh > 0.0f) & (sw > 0.0f) & (sh < (float)(Hs - 1)) & (sw < (float)(Ws - 1));
  const int fh = ok ? (int)sh : 0;
  const int fw = ok ? (int)sw : 0;
  dh = ok ? xsub(sh, (float)fh) : 0.0f;
  dw = ok ? xsub(sw, (float)fw) : 0.0f;
  return ok ? fw + Ws * (fh + c.row0) : -1;
}

// Shared memory per warp of the plane-major forward: one 16-byte record and one texel index per (view, lane),
// three ballot words per view / block.
__host__ __device__ inline size_t pm_fwd_smem_per_warp(int NV) {
  return (size_t)NV * 32 * 16 + (size_t)NV * 32 * 4 + 16;
}

// five 128-thread CTAs per SM (96 registers, 12 bytes of spill) measured fastest at c1: 120 us; six (80 registers,
// 72 bytes spilled) 124 us; three 256-thread CTAs 126 us; seven and more spill heavily (130 us and up)
#ifndef CHOP_PM_FWD_WARPS
#define CHOP_PM_FWD_WARPS 4
#endif
#ifndef CHOP_PM_FWD_BLOCKS
#define CHOP_PM_FWD_BLOCKS 5
#endif

// AGG = true is CostAggregate MEAN (cost_aggregate_kernels_gpu.cu.cc:34-127): the voxel's cost is the sum of the C
// squared differences divided by views*C.  A lane keeps the sum over its four channels per plane of the block; after
// the block the LG lanes of a pixel reduce-scatter those partials (lane li ends up with plane li) and store one float
// each - LG consecutive floats per pixel.
template <typename T, int C, int NV, bool AGG = false>
__global__ void __launch_bounds__(32 * CHOP_PM_FWD_WARPS, CHOP_PM_FWD_BLOCKS) cv_fwd_pm(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LG = C / 4;
  constexpr int G = 32 / LG;
  static_assert(LG * 4 == C && (LG & (LG - 1)) == 0 && LG >= 2 && LG <= 8, "C in {8, 16, 32}");
  static_assert(NV >= 1 && NV <= 2, "the footprints of all views live in registers");
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int li = lane & (LG - 1);
  const int g = lane / LG;

  const long long item = (long long)blockIdx.x * warps + wib;
  if (item >= (long long)a.npb * a.nchunks) return;
  const int chunk_id = (int)(item / a.npb);
  const int pb = (int)(item - (long long)chunk_id * a.npb);
  const long long pix0 = (long long)pb * G;
  const bool pvalid = pix0 + g < a.npix;
  const long long pix = pvalid ? pix0 + g : a.npix - 1;
  const int dlo = a.d_begin + chunk_id * a.chunk;
  const int dhi = min(a.d_end, dlo + a.chunk);
  const int D = a.D;

  unsigned char* mine = smem_raw + (size_t)wib * smem_per_warp;
  float4* rec = reinterpret_cast<float4*>(mine);               // [NV][32] {dw, dw, dh, dh}
  int* tex = reinterpret_cast<int*>(rec + NV * 32);            // [NV][32] top-left texel or -1
  unsigned* flg = reinterpret_cast<unsigned*>(tex + NV * 32);  // [0..NV): footprint changes at plane j; [NV]: every view sees it

  // this lane's pixel: row products of every view (cost_volume_kernels_gpu.cu.cc:65-70,83,88,91), reference pixel
  Coef<float> cf[NV];
  {
    const int w = (int)(pix % a.W);
    const long long tt = pix / a.W;
    const int h = (int)(tt % a.H);
    const int bb = (int)(tt / a.H);
    float x = (float)w, y = (float)h;
    if (a.half_centor) {
      x = xadd(x, 0.5f);
      y = xadd(y, 0.5f);
    }
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const float* Rm = static_cast<const float*>(a.Rs) + (size_t)(bb * NV + n) * 9;
      const float* tv = static_cast<const float*>(a.Ts) + (size_t)(bb * NV + n) * 3;
      cf[n].zc = xadd(xadd(xmul(Rm[6], x), xmul(Rm[7], y)), Rm[8]);
      cf[n].wc = xadd(xadd(xmul(Rm[0], x), xmul(Rm[1], y)), Rm[2]);
      cf[n].hc = xadd(xadd(xmul(Rm[3], x), xmul(Rm[4], y)), Rm[5]);
      cf[n].t0 = tv[0];
      cf[n].t1 = tv[1];
      cf[n].t2 = tv[2];
      cf[n].row0 = a.Hs * (n + NV * bb);
    }
  }
  const T* src_lane = static_cast<const T*>(a.src) + li * 4;
  const T* ref_lane = static_cast<const T*>(a.ref) + pix * C + li * 4;
  pk2 ref0, ref1;
  PkLoad<T>::ld(ref_lane, ref0, ref1);
  const int b = (int)(pix / ((long long)a.H * a.W));
  const float base = static_cast<const float*>(a.depth)[pix];
  const float* offs = static_cast<const float*>(a.offsets) + (long long)b * D;
  const long long dx_bytes = (long long)C * (long long)sizeof(T);
  const long long dy_bytes = (long long)a.Ws * dx_bytes;
  float* out = AGG ? static_cast<float*>(a.cost) + pix * D + dlo + li   // one value per voxel, lane li stores plane li
                   : static_cast<float*>(a.cost) + (pix * D + dlo) * C + li * 4;
  const ulonglong2* rec_mine = reinterpret_cast<const ulonglong2*>(rec) + g * LG;
  const int* tex_mine = tex + g * LG;
  const pk2 half2 = pk_make(0.5f, 0.5f);

  Footprint F[NV];
  int carry[NV];  // texel of the pixel's last plane in the previous block (what the cached footprint holds)
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    F[n].a0a = F[n].a0b = F[n].ua = F[n].ub = F[n].va = F[n].vb = F[n].ta = F[n].tb = 0ull;
    carry[n] = -1;
  }

  for (int dblk = dlo; dblk < dhi; dblk += LG, out += AGG ? LG : LG * C) {
    // ---- phase A: lane (g, li) projects plane dblk+li of pixel g into every view ---------------------
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      const float depth = dv ? xadd(base, offs[d]) : 1.0f;
      int used = 0;
      int tt[NV];
      float dhh[NV], dww[NV];
#pragma unroll
      for (int n = 0; n < NV; ++n) tt[n] = project_nb(cf[n], depth, a.half_centor, a.Hs, a.Ws, dhh[n], dww[n]);
#pragma unroll
      for (int n = 0; n < NV; ++n) {
        const int t = dv ? tt[n] : -1;
        const float dh = dv ? dhh[n] : 0.0f, dw = dv ? dww[n] : 0.0f;
        used += t >= 0;
        rec[n * 32 + lane] = make_float4(dw, dw, dh, dh);
        tex[n * 32 + lane] = t;
        int prev = __shfl_up_sync(0xffffffffu, t, 1);
        if (li == 0) prev = carry[n];
        const unsigned bal = __ballot_sync(0xffffffffu, t != prev);
        if (lane == 0) flg[n] = bal;
        carry[n] = __shfl_sync(0xffffffffu, t, g * LG + LG - 1);
      }
      if (dv) __stcs(a.mask + pix * D + d, used);
      if (NV == 2) {
        const unsigned both = __ballot_sync(0xffffffffu, used == 2);
        if (lane == 0) flg[NV] = both;
      }
    }
    __syncwarp();

    // ---- phase B ---------------------------------------------------------------------------------------
    float part[AGG ? LG : 1];   // AGG: the lane's channel sum per plane of the block
#pragma unroll
    for (int j = 0; j < (AGG ? LG : 1); ++j) part[j] = 0.0f;
    if (pvalid) {
      unsigned m[NV], many = 0u;
#pragma unroll
      for (int n = 0; n < NV; ++n) {
        m[n] = flg[n] >> (g * LG);
        many |= m[n];
      }
      const unsigned both = NV == 2 ? flg[NV] >> (g * LG) : 0u;
      const int left = dhi - dblk;
      ulonglong2 whn[NV];   // the records of the next plane, requested one plane ahead
#pragma unroll
      for (int n = 0; n < NV; ++n) whn[n] = rec_mine[n * 32];
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        ulonglong2 whc[NV];
#pragma unroll
        for (int n = 0; n < NV; ++n) {
          whc[n] = whn[n];
          if (j + 1 < LG) whn[n] = rec_mine[n * 32 + j + 1];
        }
        if ((many >> j) & 1u) {  // some view's footprint moves at this plane (one test per plane on the common path)
#pragma unroll
          for (int n = 0; n < NV; ++n) {
            if ((m[n] >> j) & 1u) {
              const int t = tex_mine[n * 32 + j];
              // the empty footprint (the view does not see the plane): four reads of the reference pixel
              const T* p = t >= 0 ? src_lane + (size_t)t * C : ref_lane;
              FootprintLoad<T>::go(F[n], p, t >= 0 ? dx_bytes : 0ll, t >= 0 ? dy_bytes : 0ll, ref0, ref1);
            }
          }
        }
        pk2 acc0, acc1;
#pragma unroll
        for (int n = 0; n < NV; ++n) {
          const ulonglong2 wh = whc[n];  // x = {dw, dw}, y = {dh, dh}
          const pk2 X0 = pk_fma(F[n].ta, wh.x, F[n].ua);
          const pk2 X1 = pk_fma(F[n].tb, wh.x, F[n].ub);
          const pk2 Y0 = pk_fma(wh.x, F[n].va, F[n].a0a);
          const pk2 Y1 = pk_fma(wh.x, F[n].vb, F[n].a0b);
          const pk2 d0 = pk_fma(wh.y, X0, Y0);  // sample - ref
          const pk2 d1 = pk_fma(wh.y, X1, Y1);
          acc0 = n == 0 ? pk_mul(d0, d0) : pk_fma(d0, d0, acc0);
          acc1 = n == 0 ? pk_mul(d1, d1) : pk_fma(d1, d1, acc1);
        }
        if (NV == 2 && ((both >> j) & 1u)) {  // mean over two views; one view: the sum itself; none: an exact zero
          acc0 = pk_mul(acc0, half2);
          acc1 = pk_mul(acc1, half2);
        }
        if constexpr (AGG) {
          float s0, s1;
          pk_split(pk_add(acc0, acc1), s0, s1);
          part[j] = s0 + s1;
        } else {
          if (j < left) pk_store_stream(out + j * C, acc0, acc1);
        }
      }
    }
    if constexpr (AGG) {
      // reduce-scatter over the pixel's LG lanes: lane li keeps plane li
#pragma unroll
      for (int sft = LG / 2; sft >= 1; sft >>= 1) {
#pragma unroll
        for (int i = 0; i < sft; ++i) {
          const bool hi = (li & sft) != 0;
          const float keep = hi ? part[i + sft] : part[i];
          const float send = hi ? part[i] : part[i + sft];
          part[i] = keep + __shfl_xor_sync(0xffffffffu, send, sft);
        }
      }
      if (pvalid && dblk + li < dhi) __stcs(out, part[0] * (1.0f / (float)C));
    }
    __syncwarp();
  }
}

}  // namespace chop
