// Fused epilogues of the tcgen05 GEMMs, shared by the single-CTA kernel (gemm_tcgen05.cu) and the
// CTA-pair kernel (gemm2_tcgen05.cu).  One call drains this warp's 32 TMEM lanes (one output row
// per thread) for its half of the tile's 256 accumulator columns.
#pragma once
#include "ws_ptx.cuh"
#include "ws_api.h"

namespace ws {

constexpr int EPI_BN = 256;  // accumulator columns per tile

struct GemmParams {
  int m, n, k;
  int epi_n;  // width of one logical N tile in output columns (256, or 128 for SwiGLU)
  int h;      // SwiGLU half width
  void* out;
  int ldo;
  void* out2;
  int ldo2;
  const void* aux;
  int ldaux;
  const float* row_scale;
  const float* row_vec;
  float alpha, beta;
  int* error_flag;
  int debug;  // experiment switch: 1 = no loads (MMA issue rate only), 2 = always load tile (0,0)
};

__device__ __forceinline__ float sigmoidf_(float x) { return sigmoid_fast(x); }

// taddr: TMEM address of (this warp's first lane, first column of the accumulator buffer).
// row: global output row of this thread; nb: N-tile index; egroup: which half of the columns.
// GROUPS: how many warpgroups of four warps share a tile's columns (egroup in [0, GROUPS)).
// Two everywhere: four groups on the SwiGLU epilogues measured 5-10 % slower (their
// row-per-thread global accesses are bound by L1 wavefronts, which more warps do not add).
template <int EPI>
constexpr int epilogue_groups() {
  return 2;
}

template <int EPI, int GROUPS = 2>
__device__ __forceinline__ void gemm_epilogue(const GemmParams& p, uint32_t taddr, int row, bool row_ok, float rs,
                                              int nb, int egroup) {
  constexpr int BN = EPI_BN;
  static_assert(GROUPS == 2 || EPI == WS_EPI_SWIGLU || EPI == WS_EPI_SWIGLU_BWD, "only the SwiGLU epilogues take 4 groups");
  if constexpr (EPI == WS_EPI_BF16) {
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ldo;
    const int n0 = nb * BN;
#pragma unroll 1
    for (int c = egroup * 128; c < egroup * 128 + 128; c += 32) {
      if (n0 + c >= p.n) break;
      uint32_t r[32];
      tmem_ld_32x32b_x32(taddr + c, r);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (n0 + c + j < p.n) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[j + 0]) * rs, __uint_as_float(r[j + 1]) * rs);
            v.y = pack_bf16x2(__uint_as_float(r[j + 2]) * rs, __uint_as_float(r[j + 3]) * rs);
            v.z = pack_bf16x2(__uint_as_float(r[j + 4]) * rs, __uint_as_float(r[j + 5]) * rs);
            v.w = pack_bf16x2(__uint_as_float(r[j + 6]) * rs, __uint_as_float(r[j + 7]) * rs);
            *reinterpret_cast<uint4*>(out + n0 + c + j) = v;
          }
        }
      }
    }
  } else if constexpr (EPI == WS_EPI_RESID_F32 || EPI == WS_EPI_ACC_F32 || EPI == WS_EPI_F32) {
    float* out = reinterpret_cast<float*>(p.out) + static_cast<size_t>(row) * p.ldo;
    const float* res = reinterpret_cast<const float*>(p.aux) + static_cast<size_t>(row) * p.ldaux;
    const int n0 = nb * BN;
#pragma unroll 1
    for (int c = egroup * 128; c < egroup * 128 + 128; c += 32) {
      if (n0 + c >= p.n) break;
      uint32_t r[32];
      tmem_ld_32x32b_x32(taddr + c, r);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          if (n0 + c + j < p.n) {
            float4 v;
            v.x = __uint_as_float(r[j + 0]);
            v.y = __uint_as_float(r[j + 1]);
            v.z = __uint_as_float(r[j + 2]);
            v.w = __uint_as_float(r[j + 3]);
            if constexpr (EPI == WS_EPI_RESID_F32) {
              const float4 q = *reinterpret_cast<const float4*>(res + n0 + c + j);
              v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
            } else if constexpr (EPI == WS_EPI_ACC_F32) {
              v.x *= p.alpha; v.y *= p.alpha; v.z *= p.alpha; v.w *= p.alpha;
              if (p.beta != 0.0f) {
                const float4 q = *reinterpret_cast<const float4*>(out + n0 + c + j);
                v.x += p.beta * q.x; v.y += p.beta * q.y; v.z += p.beta * q.z; v.w += p.beta * q.w;
              }
            }
            *reinterpret_cast<float4*>(out + n0 + c + j) = v;
          }
        }
      }
    }
  } else if constexpr (EPI == WS_EPI_RESID_BF16) {
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ldo;
    const __nv_bfloat16* res =
        reinterpret_cast<const __nv_bfloat16*>(p.aux) + static_cast<size_t>(row) * p.ldaux;
    const int n0 = nb * BN;
#pragma unroll 1
    for (int c = egroup * 128; c < egroup * 128 + 128; c += 32) {
      if (n0 + c >= p.n) break;
      uint32_t r[32];
      tmem_ld_32x32b_x32(taddr + c, r);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (n0 + c + j < p.n) {
            const uint4 q = *reinterpret_cast<const uint4*>(res + n0 + c + j);
            const __nv_bfloat162* qb = reinterpret_cast<const __nv_bfloat162*>(&q);
            uint4 v;
            uint32_t* vw = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float2 f = __bfloat1622float2(qb[t]);
              vw[t] = pack_bf16x2(f.x + bf16_round(__uint_as_float(r[j + 2 * t])),
                                  f.y + bf16_round(__uint_as_float(r[j + 2 * t + 1])));
            }
            *reinterpret_cast<uint4*>(out + n0 + c + j) = v;
          }
        }
      }
    }
  } else if constexpr (EPI == WS_EPI_SWIGLU) {
    // Accumulator columns 0..127 are `up`, 128..255 are `gate` of the same 128 features.
    // Both halves are rounded to BF16 first (what a BF16 GEMM would have returned); the
    // activation is computed in FP32 from the rounded values and rounded once.
    __nv_bfloat16* packed = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ldo;
    __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(p.out2) + static_cast<size_t>(row) * p.ldo2;
    const int n0 = nb * 128;
    constexpr int GW = 128 / GROUPS;
#pragma unroll 1
    for (int c = egroup * GW; c < egroup * GW + GW; c += 16) {
      if (n0 + c >= p.h) break;
      uint32_t ru[16], rg[16];
      tmem_ld_32x32b_x16(taddr + c, ru);
      tmem_ld_32x32b_x16(taddr + 128 + c, rg);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 16; j += 8) {
          if (n0 + c + j < p.h) {
            uint4 vu, vg, va;
            uint32_t* wu = reinterpret_cast<uint32_t*>(&vu);
            uint32_t* wg = reinterpret_cast<uint32_t*>(&vg);
            uint32_t* wa = reinterpret_cast<uint32_t*>(&va);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float u0 = bf16_round(__uint_as_float(ru[j + 2 * t]) * rs);
              const float u1 = bf16_round(__uint_as_float(ru[j + 2 * t + 1]) * rs);
              const float g0 = bf16_round(__uint_as_float(rg[j + 2 * t]) * rs);
              const float g1 = bf16_round(__uint_as_float(rg[j + 2 * t + 1]) * rs);
              wu[t] = pack_bf16x2(u0, u1);
              wg[t] = pack_bf16x2(g0, g1);
              wa[t] = pack_bf16x2(g0 * sigmoidf_(g0) * u0, g1 * sigmoidf_(g1) * u1);
            }
            if (p.out != nullptr) {
              *reinterpret_cast<uint4*>(packed + n0 + c + j) = vu;
              *reinterpret_cast<uint4*>(packed + p.h + n0 + c + j) = vg;
            }
            *reinterpret_cast<uint4*>(act + n0 + c + j) = va;
          }
        }
      }
    }
  } else if constexpr (EPI == WS_EPI_SWIGLU_BWD) {
    // acc = dAct; aux = packed (up|gate) of the forward; out = packed (dUp|dGate).
    // The (up, gate) values of the next 16 columns are requested before the current 16 are
    // processed, so their global-load latency overlaps the TMEM read and the arithmetic.
    __nv_bfloat16* dpk = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ldo;
    const __nv_bfloat16* pk =
        reinterpret_cast<const __nv_bfloat16*>(p.aux) + static_cast<size_t>(row) * p.ldaux;
    const int n0 = nb * BN;
    constexpr int GWB = BN / GROUPS;
    const int c_end = egroup * GWB + GWB;
    uint4 cu[2], cg[2], nu[2], ng[2];
    auto load_aux = [&](int c, uint4(&u)[2], uint4(&g)[2]) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        if (row_ok && n0 + c + q * 8 < p.n) {
          u[q] = *reinterpret_cast<const uint4*>(pk + n0 + c + q * 8);
          g[q] = *reinterpret_cast<const uint4*>(pk + p.n + n0 + c + q * 8);
        } else {
          u[q] = make_uint4(0u, 0u, 0u, 0u);
          g[q] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    };
    load_aux(egroup * GWB, cu, cg);
#pragma unroll 1
    for (int c = egroup * GWB; c < c_end; c += 16) {
      if (n0 + c >= p.n) break;
      uint32_t r[16];
      tmem_ld_32x32b_x16(taddr + c, r);
      if (c + 16 < c_end) load_aux(c + 16, nu, ng);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 16; j += 8) {
          if (n0 + c + j < p.n) {
            const __nv_bfloat162* bu = reinterpret_cast<const __nv_bfloat162*>(&cu[j >> 3]);
            const __nv_bfloat162* bg = reinterpret_cast<const __nv_bfloat162*>(&cg[j >> 3]);
            uint4 vu, vg;
            uint32_t* wu = reinterpret_cast<uint32_t*>(&vu);
            uint32_t* wg = reinterpret_cast<uint32_t*>(&vg);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float2 u = __bfloat1622float2(bu[t]);
              const float2 g = __bfloat1622float2(bg[t]);
              const float d0 = bf16_round(__uint_as_float(r[j + 2 * t]));
              const float d1 = bf16_round(__uint_as_float(r[j + 2 * t + 1]));
              const float s0 = sigmoidf_(g.x), s1 = sigmoidf_(g.y);
              wu[t] = pack_bf16x2(d0 * g.x * s0, d1 * g.y * s1);
              wg[t] = pack_bf16x2(d0 * u.x * s0 * (1.0f + g.x * (1.0f - s0)),
                                  d1 * u.y * s1 * (1.0f + g.y * (1.0f - s1)));
            }
            *reinterpret_cast<uint4*>(dpk + n0 + c + j) = vu;
            *reinterpret_cast<uint4*>(dpk + p.n + n0 + c + j) = vg;
          }
        }
      }
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        cu[q] = nu[q];
        cg[q] = ng[q];
      }
    }
  } else if constexpr (EPI == WS_EPI_CE_FWD) {
    // LM head forward: the logits tile never leaves the SM.  Each thread folds its 128
    // columns of one row into (max, sum exp) and the owner of the label column records the
    // label's logit.  Logits are rounded to BF16 first, as a BF16 head GEMM would return them.
    const long long* labels = reinterpret_cast<const long long*>(p.aux);
    const long long lab = row_ok ? labels[row] : -1;
    const int n0 = nb * BN;
    float mx = -INFINITY, sm = 0.f;
#pragma unroll 1
    for (int c = egroup * 128; c < egroup * 128 + 128; c += 32) {
      if (n0 + c >= p.n) break;
      uint32_t r[32];
      tmem_ld_32x32b_x32(taddr + c, r);
      tmem_ld_wait();
      float cm = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float v = (n0 + c + j < p.n) ? bf16_round(__uint_as_float(r[j])) : -INFINITY;
        r[j] = __float_as_uint(v);
        cm = fmaxf(cm, v);
        if (n0 + c + j == lab) reinterpret_cast<float*>(p.out2)[row] = v;
      }
      const float nm = fmaxf(mx, cm);
      float cs = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) cs += __expf(__uint_as_float(r[j]) - nm);
      sm = sm * __expf(mx - nm) + cs;
      mx = nm;
    }
    if (row_ok && n0 + egroup * 128 < p.n) {
      float2* part = reinterpret_cast<float2*>(p.out) + static_cast<size_t>(row) * p.ldo + (nb * 2 + egroup);
      *part = make_float2(mx, sm);
    }
  } else if constexpr (EPI == WS_EPI_CE_BWD) {
    // LM head backward: recompute the logits tile and emit
    // dlogits = (softmax - onehot(label)) * row_weight in BF16.
    const long long* labels = reinterpret_cast<const long long*>(p.aux);
    const long long lab = row_ok ? labels[row] : -1;
    const float lse = row_ok ? p.row_vec[row] : 0.f;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ldo;
    const int n0 = nb * BN;
#pragma unroll 1
    for (int c = egroup * 128; c < egroup * 128 + 128; c += 32) {
      if (n0 + c >= p.n) break;
      uint32_t r[32];
      tmem_ld_32x32b_x32(taddr + c, r);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (n0 + c + j < p.n) {
            uint4 v;
            uint32_t* vw = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const int col = n0 + c + j + 2 * t;
              float d0 = __expf(bf16_round(__uint_as_float(r[j + 2 * t])) - lse);
              float d1 = __expf(bf16_round(__uint_as_float(r[j + 2 * t + 1])) - lse);
              if (col == lab) d0 -= 1.f;
              if (col + 1 == lab) d1 -= 1.f;
              vw[t] = pack_bf16x2(d0 * rs, d1 * rs);
            }
            *reinterpret_cast<uint4*>(out + n0 + c + j) = v;
          }
        }
      }
    }
  }
}

}  // namespace ws
