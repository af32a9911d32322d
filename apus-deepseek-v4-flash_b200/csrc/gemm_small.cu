// Small-M block-scaled GEMM: the decode GEMV / expert-group kernel.
//
// out[m, o] for up to 32 activation rows per work item, streaming each weight
// matrix from HBM exactly once.  HBM-bound by design: algorithmic bytes per
// work item = O*K/2 + O*K/32 (MXFP4) or O*K + tile scales (FP8).
//
// Numerics follow the reference's normative path:
//   MXFP4 (reference c/fp4.h:367-395): per 32-wide K block the dot of E4M3
//     activation codes and E2M1 weight values, then
//     total += (dot * act_scale[m, kb/4]) * 2^(wscale[o, kb] - 127), kb ascending.
//   FP8 (reference c/fp8.h:191-218): per 128-wide K block the dot of E4M3 x E4M3,
//     then total += dot * (act_scale[m, kb] * 2^(wscale[o/128, kb] - 127)).
// The block dots run on the tensor cores (mma.sync m16n8k32 E4M3 x E4M3 -> f32;
// E2M1 values are expanded to E4M3 bytes, which is exact); the products are
// exact and the scales are powers of two, so the only difference from the
// reference's sequential f32 dot is the summation order inside a block.
// The fold over blocks keeps the reference's kb order.
//
// Pair mode computes gate = A x and up = B x for the same rows and writes
// h = bf16(silu(clamp(gate)) * clamp(up)) (reference c/moe.h:113-126) so the
// gate/up projections of an expert cost one pass over the activations.
//
// Launch, MXFP4: grid (ceil(O/128), work items), 256 threads; warp w of a CTA owns
// the 16 output rows [blockIdx.x*128 + 16w, +16) for the whole K range (the fold
// over K blocks keeps the reference order) and reads its weight fragments
// straight from global memory in the tiled layout of repack.cu (coalesced 16
// bytes per lane); activation codes of the work item's rows are staged once in
// shared memory.
// Launch, FP8 (dense projections, shared expert: one matrix, few work items):
// grid (O/16, work items); the 8 warps of a CTA share one 16-row group and split
// K into eight contiguous ranges, their partial totals are added in warp order
// through shared memory.  The split does not depend on the number of rows, so
// a row's result is the same in any batch.
#include "common.cuh"
#include "kernels.cuh"

namespace apus {

__device__ __forceinline__ void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1,
                                         uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1, const float (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1),
          "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// Eight re-encoded E2M1 elements -> two registers of four E4M3 bytes
// (elements 0..3 and 4..7 of the lane's K slice); see repack.cu.
__device__ __forceinline__ void fp4_expand(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t T0 = 0x3C383000u;   // E4M3 codes of 0, .5, 1, 1.5
    const uint32_t T1 = 0x4C484440u;   // E4M3 codes of 2, 3, 4, 6
    uint32_t m = w & 0x77777777u;
    lo = __byte_perm(T0, T1, m) | (w & 0x80808080u);
    hi = __byte_perm(T0, T1, m >> 16) | ((w << 4) & 0x80808080u);
}

__device__ __forceinline__ float swiglu(float gate, float up, float limit) {
    float g = bf16_round(gate), u = bf16_round(up);
    if (limit > 0.f) {
        u = fminf(fmaxf(u, -limit), limit);
        g = fminf(g, limit);
    }
    float sig = 1.0f / (1.0f + exp_rn(-g));
    return bf16_round(__fmul_rn(__fmul_rn(g, sig), u));
}

template <bool ZS>
__device__ __forceinline__ float wscale(uint32_t word, int b) {
    uint32_t byte = (word >> (8 * b)) & 0xffu;
    if (ZS) return ue8m0_f32(byte);
    return __uint_as_float(byte << 23);
}

template <int FMT, int NT, bool PAIR, bool ZS>
__global__ void __launch_bounds__(256, (NT <= 2 ? 2 : 1))
gemm_small_kernel(const GemmSmallArgs a) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ __align__(16) uint8_t smem[];
    const int K = a.K, O = a.O, KG = K >> 7;
    const int pitch = K + 32;               // +32 B: bank-conflict-free 8-byte reads
    uint8_t *s_codes = smem;
    float *s_as = reinterpret_cast<float *>(smem + (size_t)NT * 8 * pitch);

    int n_groups = a.n_groups_dev ? *a.n_groups_dev : a.n_groups;
    if ((int)blockIdx.y >= n_groups) return;
    const GemmGroup grp = a.groups[blockIdx.y];
    const int nrows = grp.nrows, row0 = grp.row0;
    if (nrows <= 0) return;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    constexpr bool SPLITK = (FMT == 8);
    const int rg = SPLITK ? (int)blockIdx.x : (int)blockIdx.x * 8 + warp;
    const bool active = rg * 16 < O;
    const int kg_lo = SPLITK ? (KG * warp) / 8 : 0;
    const int kg_hi = SPLITK ? (KG * (warp + 1)) / 8 : KG;

    // ---- weight stream pointers ------------------------------------------------
    const uint4 *pa = nullptr, *pb = nullptr;
    const uint2 *qa = nullptr, *qb = nullptr;       // MXFP4 scale words
    const uint8_t *ta = nullptr, *tb = nullptr;     // FP8 tile scale rows
    if (active) {
        if (FMT == 4) {
            pa = reinterpret_cast<const uint4 *>(grp.wa) + (size_t)rg * (K / 64) * 32 + lane;
            qa = reinterpret_cast<const uint2 *>(grp.sa) + (size_t)rg * KG * 8 + g;
            if (PAIR) {
                pb = reinterpret_cast<const uint4 *>(grp.wb) + (size_t)rg * (K / 64) * 32 + lane;
                qb = reinterpret_cast<const uint2 *>(grp.sb) + (size_t)rg * KG * 8 + g;
            }
        } else {
            pa = reinterpret_cast<const uint4 *>(grp.wa) + (size_t)rg * (K / 32) * 32 + lane;
            ta = grp.sa + (size_t)(rg >> 3) * KG;
            if (PAIR) {
                pb = reinterpret_cast<const uint4 *>(grp.wb) + (size_t)rg * (K / 32) * 32 + lane;
                tb = grp.sb + (size_t)(rg >> 3) * KG;
            }
        }
    }
    constexpr int NW = (FMT == 4) ? 2 : 4;          // 16-byte loads per 128-wide K group
    uint4 wa[NW], wb[NW];
    uint2 sa = make_uint2(0, 0), sb = make_uint2(0, 0);
    auto load_group = [&](int kg, uint4 (&xa)[NW], uint4 (&xb)[NW], uint2 &ya, uint2 &yb) {
#pragma unroll
        for (int i = 0; i < NW; i++) {
            xa[i] = __ldg(pa + ((size_t)kg * NW + i) * 32);
            if (PAIR) xb[i] = __ldg(pb + ((size_t)kg * NW + i) * 32);
        }
        if (FMT == 4) {
            ya = __ldg(qa + (size_t)kg * 8);
            if (PAIR) yb = __ldg(qb + (size_t)kg * 8);
        } else {
            ya.x = ta[kg];
            if (PAIR) yb.x = tb[kg];
        }
    };
    if (active && kg_lo < kg_hi) load_group(kg_lo, wa, wb, sa, sb);   // in flight while activations stage

    // ---- stage activation codes + scales of this work item ------------------------
    {
        const int chunks = K >> 4;
        for (int i = tid; i < NT * 8 * chunks; i += 256) {
            int r = i / chunks, ch = i - r * chunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < nrows) {
                int src = a.arow ? a.arow[row0 + r] : row0 + r;
                v = *reinterpret_cast<const uint4 *>(a.acodes + (size_t)src * K + ch * 16);
            }
            *reinterpret_cast<uint4 *>(s_codes + (size_t)r * pitch + ch * 16) = v;
        }
        for (int i = tid; i < NT * 8 * KG; i += 256) {
            int r = i / KG, kg = i - r * KG;
            float v = 0.f;
            if (r < nrows) {
                int src = a.arow ? a.arow[row0 + r] : row0 + r;
                v = a.ascales[(size_t)src * KG + kg];
            }
            s_as[kg * (NT * 8) + r] = v;
        }
    }
    __syncthreads();
    if (!active) return;

    float totA[NT][4], totB[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int j = 0; j < 4; j++) { totA[nt][j] = 0.f; totB[nt][j] = 0.f; }
    const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
    const uint8_t *bbase = s_codes + (size_t)g * pitch + 8 * c;

    for (int kg = kg_lo; kg < kg_hi; kg++) {
        uint4 na[NW], nb[NW];
        uint2 nsa = make_uint2(0, 0), nsb = make_uint2(0, 0);
        if (kg + 1 < kg_hi) load_group(kg + 1, na, nb, nsa, nsb);

        float2 as2[NT];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
            as2[nt] = *reinterpret_cast<const float2 *>(s_as + kg * (NT * 8) + nt * 8 + 2 * c);

        if (FMT == 4) {
#pragma unroll
            for (int b = 0; b < 4; b++) {
                uint32_t wg = (b & 1) ? wa[b >> 1].z : wa[b >> 1].x;
                uint32_t wh = (b & 1) ? wa[b >> 1].w : wa[b >> 1].y;
                uint32_t a0, a1, a2, a3;
                fp4_expand(wg, a0, a2);
                fp4_expand(wh, a1, a3);
                float sg = wscale<ZS>(sa.x, b), sh = wscale<ZS>(sa.y, b);
                uint32_t e0 = 0, e1 = 0, e2 = 0, e3 = 0;
                float tg = 0.f, th = 0.f;
                if (PAIR) {
                    uint32_t vg = (b & 1) ? wb[b >> 1].z : wb[b >> 1].x;
                    uint32_t vh = (b & 1) ? wb[b >> 1].w : wb[b >> 1].y;
                    fp4_expand(vg, e0, e2);
                    fp4_expand(vh, e1, e3);
                    tg = wscale<ZS>(sb.x, b);
                    th = wscale<ZS>(sb.y, b);
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    uint2 bf = *reinterpret_cast<const uint2 *>(
                        bbase + (size_t)nt * 8 * pitch + (kg * 4 + b) * 32);
                    float d[4];
                    mma_e4m3(d, a0, a1, a2, a3, bf.x, bf.y, zero4);
                    totA[nt][0] = fmaf(__fmul_rn(d[0], as2[nt].x), sg, totA[nt][0]);
                    totA[nt][1] = fmaf(__fmul_rn(d[1], as2[nt].y), sg, totA[nt][1]);
                    totA[nt][2] = fmaf(__fmul_rn(d[2], as2[nt].x), sh, totA[nt][2]);
                    totA[nt][3] = fmaf(__fmul_rn(d[3], as2[nt].y), sh, totA[nt][3]);
                    if (PAIR) {
                        mma_e4m3(d, e0, e1, e2, e3, bf.x, bf.y, zero4);
                        totB[nt][0] = fmaf(__fmul_rn(d[0], as2[nt].x), tg, totB[nt][0]);
                        totB[nt][1] = fmaf(__fmul_rn(d[1], as2[nt].y), tg, totB[nt][1]);
                        totB[nt][2] = fmaf(__fmul_rn(d[2], as2[nt].x), th, totB[nt][2]);
                        totB[nt][3] = fmaf(__fmul_rn(d[3], as2[nt].y), th, totB[nt][3]);
                    }
                }
            }
        } else {
            float ws_a = ue8m0_f32(sa.x & 0xffu);
            float ws_b = PAIR ? ue8m0_f32(sb.x & 0xffu) : 0.f;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                float dA[4] = {0.f, 0.f, 0.f, 0.f}, dB[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    uint2 bf = *reinterpret_cast<const uint2 *>(
                        bbase + (size_t)nt * 8 * pitch + (kg * 4 + b) * 32);
                    mma_e4m3(dA, wa[b].x, wa[b].y, wa[b].z, wa[b].w, bf.x, bf.y, dA);
                    if (PAIR) mma_e4m3(dB, wb[b].x, wb[b].y, wb[b].z, wb[b].w, bf.x, bf.y, dB);
                }
                float s0 = __fmul_rn(as2[nt].x, ws_a), s1 = __fmul_rn(as2[nt].y, ws_a);
                totA[nt][0] = fmaf(dA[0], s0, totA[nt][0]);
                totA[nt][1] = fmaf(dA[1], s1, totA[nt][1]);
                totA[nt][2] = fmaf(dA[2], s0, totA[nt][2]);
                totA[nt][3] = fmaf(dA[3], s1, totA[nt][3]);
                if (PAIR) {
                    float u0 = __fmul_rn(as2[nt].x, ws_b), u1 = __fmul_rn(as2[nt].y, ws_b);
                    totB[nt][0] = fmaf(dB[0], u0, totB[nt][0]);
                    totB[nt][1] = fmaf(dB[1], u1, totB[nt][1]);
                    totB[nt][2] = fmaf(dB[2], u0, totB[nt][2]);
                    totB[nt][3] = fmaf(dB[3], u1, totB[nt][3]);
                }
            }
        }
        if (kg + 1 < kg_hi) {
#pragma unroll
            for (int i = 0; i < NW; i++) { wa[i] = na[i]; if (PAIR) wb[i] = nb[i]; }
            sa = nsa; sb = nsb;
        }
    }

    if (SPLITK) {
        // add the eight K-range partials in warp order (the staging area is free now)
        __syncthreads();
        float *part = reinterpret_cast<float *>(smem);
        constexpr int PER = NT * 4 * (PAIR ? 2 : 1);
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                part[(warp * PER + nt * 4 + j) * 32 + lane] = totA[nt][j];
                if (PAIR) part[(warp * PER + NT * 4 + nt * 4 + j) * 32 + lane] = totB[nt][j];
            }
        __syncthreads();
        if (warp != 0) return;
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float a0 = 0.f, b0 = 0.f;
#pragma unroll
                for (int w = 0; w < 8; w++) {
                    a0 += part[(w * PER + nt * 4 + j) * 32 + lane];
                    if (PAIR) b0 += part[(w * PER + NT * 4 + nt * 4 + j) * 32 + lane];
                }
                totA[nt][j] = a0; totB[nt][j] = b0;
            }
    }

    // ---- epilogue ------------------------------------------------------------------
    const int o_g = rg * 16 + g;
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int col = nt * 8 + 2 * c + (j & 1);
            if (col >= nrows) continue;
            int o = o_g + ((j & 2) ? 8 : 0);
            int dst = a.orow ? a.orow[row0 + col] : row0 + col;
            float v;
            if (PAIR) v = swiglu(totA[nt][j], totB[nt][j], a.limit);
            else v = a.round_out ? bf16_round(totA[nt][j]) : totA[nt][j];
            a.out[(size_t)dst * O + o] = v;
        }
}

template <int FMT, int NT, bool PAIR, bool ZS>
static int launch(const GemmSmallArgs &a, cudaStream_t st) {
    size_t smem = (size_t)NT * 8 * (a.K + 32) + (size_t)(a.K / 128) * NT * 8 * sizeof(float);
    if (FMT == 8) {                       // the split-K partials reuse the staging area
        size_t part = (size_t)8 * NT * 4 * (PAIR ? 2 : 1) * 32 * sizeof(float);
        if (part > smem) smem = part;
    }
    auto kern = gemm_small_kernel<FMT, NT, PAIR, ZS>;
    if (ensure_dyn_smem((const void *)kern, smem)) return 1;
    dim3 grid((unsigned)(FMT == 8 ? a.O / 16 : ceil_div(a.O, 128)), (unsigned)a.n_groups);
    launch_k(kern, grid, 256, smem, st, a);
    APUS_LAUNCHED();
    return 0;
}

template <int FMT, bool PAIR, bool ZS>
static int pick_nt(const GemmSmallArgs &a, cudaStream_t st) {
    if (a.max_rows <= 8) return launch<FMT, 1, PAIR, ZS>(a, st);
    if (a.max_rows <= 16) return launch<FMT, 2, PAIR, ZS>(a, st);
    return launch<FMT, 4, PAIR, ZS>(a, st);
}

int gemm_small(const GemmSmallArgs &a, cudaStream_t st) {
    APUS_REQUIRE(a.K % 128 == 0 && a.O % 16 == 0, "gemm_small: unsupported shape O=%d K=%d", a.O, a.K);
    APUS_REQUIRE(a.max_rows >= 1 && a.max_rows <= 32, "gemm_small: max_rows=%d out of range", a.max_rows);
    APUS_REQUIRE((size_t)32 * (a.K + 32) + (size_t)(a.K / 128) * 128 <= 220 * 1024,
                 "gemm_small: K=%d too large for the activation stage", a.K);
    if (a.n_groups <= 0) return 0;
    if (a.fmt == 4) {
        if (a.pair) return a.zero_scale ? pick_nt<4, true, true>(a, st) : pick_nt<4, true, false>(a, st);
        return a.zero_scale ? pick_nt<4, false, true>(a, st) : pick_nt<4, false, false>(a, st);
    }
    if (a.fmt == 8) {
        if (a.pair) return pick_nt<8, true, false>(a, st);
        return pick_nt<8, false, false>(a, st);
    }
    set_error("gemm_small: fmt=%d", a.fmt);
    return 1;
}

}  // namespace apus
