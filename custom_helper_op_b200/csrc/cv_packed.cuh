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
// The first source view is peeled: its squared difference starts the accumulators (no zero fill).
// The projection itself stays unfused and in the reference's order (cv_project.cuh), so the validity
// count is bit-exact; cost and gradients meet the float tolerances (same formulas as cv_tuned.cuh).
// Reference: custom_helper_op/cc/kernels/cost_volume_kernels_gpu.cu.cc:33-131 (forward), :342-456 (gradient).
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
// 16-byte vector reduction of two pairs into global memory.
__device__ __forceinline__ void pk_red_add(float* p, pk2 a, pk2 b) {
  asm volatile(
      "{\n\t.reg .f32 x0, x1, x2, x3;\n\t"
      "mov.b64 {x0, x1}, %1;\n\t"
      "mov.b64 {x2, x3}, %2;\n\t"
      "red.global.add.v4.f32 [%0], {x0, x1, x2, x3};\n\t}"
      ::"l"(p), "l"(a), "l"(b)
      : "memory");
}

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
  pk2 ref0, ref1;
  PkLoad<T>::ld(static_cast<const T*>(a.ref) + pix * C + li * 4, ref0, ref1);
  const int b = (int)(pix / ((long long)a.H * a.W));
  const float base = static_cast<const float*>(a.depth)[pix];
  const float* offs = static_cast<const float*>(a.offsets) + (long long)b * D;
  const size_t row = (size_t)a.Ws * C;
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
      // One view over the block's planes.  A view that does not see a plane has the "empty footprint"
      // (all differences zero): the plane then contributes exactly zero without a validity branch.
      auto view = [&](auto first_tag, const int n) {
        constexpr bool FIRST = decltype(first_tag)::value;
        const ulonglong2* r = rec_mine + n * 32;
        const int* tx = tex_mine + n * 32;
        const unsigned m = chg[n] >> (g * LG);
        pk2 a0[2], u[2], v[2], t1[2];
#pragma unroll
        for (int j = 0; j < LG; ++j) {
#ifdef CHOP_DIAG_NORELOAD
          if (j == 0) {
#else
          if (j == 0 || ((m >> j) & 1u)) {
#endif
            const int t = tx[j];
            if (t >= 0) {
              const T* p00 = src_lane + (size_t)t * C;
              const T* p10 = p00 + row;
              pk2 t00[2], t01[2], t10[2], t11[2];
              PkLoad<T>::ld(p00, t00[0], t00[1]);
              PkLoad<T>::ld(p00 + C, t01[0], t01[1]);
              PkLoad<T>::ld(p10, t10[0], t10[1]);
              PkLoad<T>::ld(p10 + C, t11[0], t11[1]);
              a0[0] = pk_sub(t00[0], ref0);
              a0[1] = pk_sub(t00[1], ref1);
#pragma unroll
              for (int k = 0; k < 2; ++k) {
                u[k] = pk_sub(t10[k], t00[k]);
                v[k] = pk_sub(t01[k], t00[k]);
                t1[k] = pk_sub(pk_sub(t11[k], t01[k]), u[k]);
              }
            } else {
#pragma unroll
              for (int k = 0; k < 2; ++k) a0[k] = u[k] = v[k] = t1[k] = 0ull;
            }
          }
          const ulonglong2 wh = r[j];  // x = {dw, dw}, y = {dh, dh}
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const pk2 X = pk_fma(t1[k], wh.x, u[k]);
            const pk2 Y = pk_fma(wh.x, v[k], a0[k]);
            const pk2 df = pk_fma(wh.y, X, Y);  // sample - ref
            acc[j][k] = FIRST ? pk_mul(df, df) : pk_fma(df, df, acc[j][k]);
          }
        }
      };
      view(std::true_type{}, 0);
      for (int n = 1; n < N; ++n) view(std::false_type{}, n);

#ifdef CHOP_DIAG_NOSTORE
      const int left = (acc[0][0] == 0x12345ull) ? dhi - dblk : 0;
#else
      const int left = dhi - dblk;
#endif
      if (left >= LG) {
#pragma unroll
        for (int j = 0; j < LG; ++j) {
          const pk2 inv = inv_mine[j];
          pk_store_stream(out + j * C, pk_mul(acc[j][0], inv), pk_mul(acc[j][1], inv));
        }
      } else {
#pragma unroll
        for (int j = 0; j < LG; ++j) {
          if (j < left) {
            const pk2 inv = inv_mine[j];
            pk_store_stream(out + j * C, pk_mul(acc[j][0], inv), pk_mul(acc[j][1], inv));
          }
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
// What limits these kernels is the SM's load-store data path (every 16 bytes a lane receives from shared
// or global memory is a quarter of a wavefront, broadcast or not), so the kernel keeps per-lane loads low:
//   * the row products of the pixel (Coef) stay in registers for the whole work item;
//   * the division by the view count needs no load: with at most two views it is a multiplication by
//     one half where both see the voxel (a ballot bit), by one otherwise (zero views give an exact zero);
//   * the reload is one asm block that updates the eight footprint registers in place; a view that does
//     not see the plane reads the reference pixel four times instead, which makes all differences zero.
// ---------------------------------------------------------------------------------------------------
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

// Shared memory per warp of the plane-major forward: one 16-byte record and one texel index per (view, lane),
// three ballot words per view / block.
__host__ __device__ inline size_t pm_fwd_smem_per_warp(int NV) {
  return (size_t)NV * 32 * 16 + (size_t)NV * 32 * 4 + 16;
}

#ifndef CHOP_PM_FWD_BLOCKS
#define CHOP_PM_FWD_BLOCKS 3
#endif

template <typename T, int C, int NV>
__global__ void __launch_bounds__(256, CHOP_PM_FWD_BLOCKS) cv_fwd_pm(const CvArgs a, const int warps, const size_t smem_per_warp) {
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
  float* out = static_cast<float*>(a.cost) + (pix * D + dlo) * C + li * 4;
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

  for (int dblk = dlo; dblk < dhi; dblk += LG, out += LG * C) {
    // ---- phase A: lane (g, li) projects plane dblk+li of pixel g into every view ---------------------
#ifdef CHOP_DIAG_NOPHASEA
    if (dblk == dlo)
#endif
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      const float depth = dv ? xadd(base, offs[d]) : 0.0f;
      int used = 0;
#pragma unroll
      for (int n = 0; n < NV; ++n) {
        int t = -1;
        float dh = 0.0f, dw = 0.0f;
        if (dv) {
          float gh, gw;
          t = project<float, false>(cf[n], depth, a.half_centor, a.Hs, a.Ws, dh, dw, gh, gw);
          used += t >= 0;
        }
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
    if (pvalid) {
      unsigned m[NV], many = 0u;
#pragma unroll
      for (int n = 0; n < NV; ++n) {
        m[n] = flg[n] >> (g * LG);
        many |= m[n];
      }
      const unsigned both = NV == 2 ? flg[NV] >> (g * LG) : 0u;
#ifdef CHOP_DIAG_NORELOAD
      if (dblk != dlo) many = 0u;
#endif
#ifdef CHOP_DIAG_NOSTORE
      const int left = (F[0].a0a == 0x12345ull) ? dhi - dblk : 0;
#else
      const int left = dhi - dblk;
#endif
#pragma unroll
      for (int j = 0; j < LG; ++j) {
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
          const ulonglong2 wh = rec_mine[n * 32 + j];  // x = {dw, dw}, y = {dh, dh}
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
        if (j < left) pk_store_stream(out + j * C, acc0, acc1);
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------------------
// gradient
//
// Per (plane, view) phase A leaves three 16-byte records
//   r1 {dw, dw, dh, dh}   r2 {gh, gh, gw, gw}   r3 {s, s, dh*dw, dh*dw}      s = 2/(views that see the voxel)
// and two ballot words per view: `vld` (the view sees the plane) and `chg` (its footprint differs from the
// previous plane's).  Per channel pair a plane costs twelve packed operations: the sample difference (3),
// the upstream factor (2), the four bilinear moments of the corner gradients (4) and the three channel
// sums behind the two coordinate derivatives (3); d(base_plane) is accumulated as a pair and folded at
// the end.  The block's slice of cost_grad is staged with cp.async as in cv_bwd_tuned.
// ---------------------------------------------------------------------------------------------------
// `vpp` = source views per pass: the records are laid out for vpp views, and a block of planes runs
// ceil(N / vpp) passes of phase A + phase B, so the shared memory per warp does not grow with N.
template <int C>
__host__ __device__ inline size_t packed_bwd_smem_per_warp(int N, int G, int vpp) {
  return (size_t)N * G * sizeof(Coef<float>) + (size_t)vpp * 32 * 48 + (size_t)vpp * 32 * 4 +
         (((size_t)vpp * 8 + 15) & ~(size_t)15) + (size_t)128 * C;
}

#ifndef CHOP_PK_BWD_BLOCKS
#define CHOP_PK_BWD_BLOCKS 6
#endif

__device__ __forceinline__ void pk_cp_async16(void* smem_dst, const void* gsrc) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}

template <typename T, int C>
__global__ void __launch_bounds__(128, CHOP_PK_BWD_BLOCKS) cv_bwd_packed(const CvArgs a, const int warps, const size_t smem_per_warp,
                                                                        const int vpp) {
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
  float4* rec = reinterpret_cast<float4*>(coef + N * G);        // [vpp][3][32]
  int* tex = reinterpret_cast<int*>(rec + vpp * 96);            // [vpp][32]
  unsigned* flg = reinterpret_cast<unsigned*>(tex + vpp * 32);  // [vpp][2]: vld, chg
  float* cgbuf = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(flg) + (((size_t)vpp * 8 + 15) & ~(size_t)15));
  float* cg_mine = cgbuf + (g * LG) * C + li * 4;               // + j*C: plane j of this pixel, this lane's channels

  stage_coefs<float>(a, coef, lane, G, pix0);

  const T* src_lane = static_cast<const T*>(a.src) + li * 4;
  float* sg_lane = static_cast<float*>(a.src_grad) + li * 4;
  pk2 ref0, ref1, rg0 = 0ull, rg1 = 0ull, dsum2 = 0ull;
  PkLoad<T>::ld(static_cast<const T*>(a.ref) + pix * C + li * 4, ref0, ref1);
  const int b = (int)(pix / ((long long)a.H * a.W));
  const float base = static_cast<const float*>(a.depth)[pix];
  const float* offs = static_cast<const float*>(a.offsets) + (long long)b * D;
  const size_t row = (size_t)a.Ws * C;
  const float* cg_src = static_cast<const float*>(a.cost_grad) + (pix * D + dlo) * C + li * 4;
  const ulonglong2* rec_mine = reinterpret_cast<const ulonglong2*>(rec) + g * LG;
  const int* tex_mine = tex + g * LG;

  // stage the first block's upstream gradient
#pragma unroll
  for (int j = 0; j < LG; ++j) {
    if (dlo + j < dhi) pk_cp_async16(cg_mine + j * C, cg_src + j * C);
    else *reinterpret_cast<float4*>(cg_mine + j * C) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");

  for (int dblk = dlo; dblk < dhi; dblk += LG, cg_src += LG * C) {
    // this lane's plane of the block: depth, and the factor 2/(views that see the voxel)
    float depth = 0.0f, scale = 0.0f;
    bool live = false;
    {
      const int d = dblk + li;
      if (pvalid && d < dhi) {
        depth = xadd(base, offs[d]);
        const int m0 = __ldg(a.mask + pix * D + d);
        live = m0 > 0;                       // cost_volume_kernels_gpu.cu.cc:367
        if (live) scale = 2.0f / (float)m0;  // :439
      }
    }
    for (int n0 = 0; n0 < N; n0 += vpp) {
      const int nn = min(vpp, N - n0);
      __syncwarp();  // the records of the previous pass / block are no longer being read
      // ---- phase A: lane (g, li) projects plane dblk+li of pixel g into the views of this pass -----------
      for (int q = 0; q < nn; ++q) {
        int t = -1;
        float dh = 0.0f, dw = 0.0f, gh = 0.0f, gw = 0.0f;
        if (live) t = project<float, true>(coef[(n0 + q) * G + g], depth, a.half_centor, a.Hs, a.Ws, dh, dw, gh, gw);
        float4* r = rec + q * 96 + lane;
        r[0] = make_float4(dw, dw, dh, dh);
        r[32] = make_float4(gh, gh, gw, gw);
        const float hw = dh * dw;
        r[64] = make_float4(scale, scale, hw, hw);
        tex[q * 32 + lane] = t;
        const int prev = __shfl_up_sync(0xffffffffu, t, 1);
        const unsigned vb = __ballot_sync(0xffffffffu, t >= 0);
        const unsigned cb = __ballot_sync(0xffffffffu, t >= 0 && (li == 0 || t != prev));
        if (lane == 0) {
          flg[2 * q] = vb;
          flg[2 * q + 1] = cb;
        }
      }
      if (n0 == 0) asm volatile("cp.async.wait_group 0;" ::: "memory");  // the slice requested a block earlier
      __syncwarp();

      // ---- phase B ---------------------------------------------------------------------------------------
      if (pvalid) {
        for (int q = 0; q < nn; ++q) {
          const ulonglong2* r = rec_mine + q * 96;
          const int* tx = tex_mine + q * 32;
          const unsigned vm = flg[2 * q] >> (g * LG);
          const unsigned cm = flg[2 * q + 1] >> (g * LG);
          int cur = -1;
          pk2 a0[2], u[2], v[2], t1[2], m0[2], m1[2], m2[2], m3[2];
#pragma unroll
          for (int k = 0; k < 2; ++k) a0[k] = u[k] = v[k] = t1[k] = m0[k] = m1[k] = m2[k] = m3[k] = 0ull;
          // moments of the per-plane sample gradients over one footprint -> its four corner gradients
          // (:441-444); the first moment is also what d(ref) loses (:440)
          auto flush = [&]() {
            float* gp = sg_lane + (size_t)cur * C;
            pk2 c00[2], c01[2], c10[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              c01[k] = pk_sub(m1[k], m3[k]);
              c10[k] = pk_sub(m2[k], m3[k]);
              c00[k] = pk_sub(pk_sub(m0[k], m1[k]), c10[k]);
            }
            rg0 = pk_sub(rg0, m0[0]);
            rg1 = pk_sub(rg1, m0[1]);
            pk_red_add(gp, c00[0], c00[1]);
            pk_red_add(gp + C, c01[0], c01[1]);
            pk_red_add(gp + row, c10[0], c10[1]);
            pk_red_add(gp + row + C, m3[0], m3[1]);
          };
#pragma unroll
          for (int j = 0; j < LG; ++j) {
            if ((vm >> j) & 1u) {
              if ((cm >> j) & 1u) {
                if (cur >= 0) flush();
                cur = tx[j];
                const T* p00 = src_lane + (size_t)cur * C;
                const T* p10 = p00 + row;
                pk2 t00[2], t01[2], t10[2], t11[2];
                PkLoad<T>::ld(p00, t00[0], t00[1]);
                PkLoad<T>::ld(p00 + C, t01[0], t01[1]);
                PkLoad<T>::ld(p10, t10[0], t10[1]);
                PkLoad<T>::ld(p10 + C, t11[0], t11[1]);
                a0[0] = pk_sub(t00[0], ref0);
                a0[1] = pk_sub(t00[1], ref1);
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                  u[k] = pk_sub(t10[k], t00[k]);
                  v[k] = pk_sub(t01[k], t00[k]);
                  t1[k] = pk_sub(pk_sub(t11[k], t01[k]), u[k]);  // :447
                  m0[k] = m1[k] = m2[k] = m3[k] = 0ull;
                }
              }
              const ulonglong2 wh = r[j];       // {dw,dw}, {dh,dh}
              const ulonglong2 gg = r[32 + j];  // {gh,gh}, {gw,gw}
              const ulonglong2 sx = r[64 + j];  // {s,s},   {dh*dw, dh*dw}
              const ulonglong2 cg = *reinterpret_cast<const ulonglong2*>(cg_mine + j * C);
              const pk2 cgv[2] = {cg.x, cg.y};
              pk2 P = 0ull, Q = 0ull, R = 0ull;
#pragma unroll
              for (int k = 0; k < 2; ++k) {
                const pk2 X = pk_fma(t1[k], wh.x, u[k]);
                const pk2 Y = pk_fma(wh.x, v[k], a0[k]);
                const pk2 df = pk_fma(wh.y, X, Y);                // sample - ref
                const pk2 gs = pk_mul(df, pk_mul(cgv[k], sx.x));  // d(cost)/d(sample) (:439)
                m0[k] = pk_add(m0[k], gs);
                m1[k] = pk_fma(gs, wh.x, m1[k]);
                m2[k] = pk_fma(gs, wh.y, m2[k]);
                m3[k] = pk_fma(gs, sx.y, m3[k]);
                if (k == 0) {
                  P = pk_mul(gs, t1[k]);
                  Q = pk_mul(gs, u[k]);
                  R = pk_mul(gs, v[k]);
                } else {
                  P = pk_fma(gs, t1[k], P);
                  Q = pk_fma(gs, u[k], Q);
                  R = pk_fma(gs, v[k], R);
                }
              }
              // coordinate derivatives (:448-449) dw*P + Q and dh*P + R, chained to the depth (:451)
              dsum2 = pk_fma(gg.x, pk_fma(wh.x, P, Q), pk_fma(gg.y, pk_fma(wh.y, P, R), dsum2));
            }
          }
          if (cur >= 0) flush();
        }
      }
    }
    // each lane has finished reading its own slots (it reads back only what it copied): request the next block's slice
    {
      const int nxt = dblk + LG;
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        if (nxt + j < dhi) pk_cp_async16(cg_mine + j * C, cg_src + (LG + j) * C);
        else *reinterpret_cast<float4*>(cg_mine + j * C) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  if (pvalid) pk_red_add(static_cast<float*>(a.ref_grad) + pix * C + li * 4, rg0, rg1);
  float dlo_f, dhi_f;
  pk_split(dsum2, dlo_f, dhi_f);
  float dsum = dlo_f + dhi_f;
#pragma unroll
  for (int o = LG >> 1; o > 0; o >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, o);
  if (pvalid && li == 0) atomicAdd(static_cast<float*>(a.depth_grad) + pix, dsum);  // :454
}

}  // namespace chop
