// FP8 (E4M3, 128x128 UE8M0 tile scales) dense GEMV/GEMM on the 5th-generation
// tensor cores (tcgen05), with the reference's fold:
//
//   out[m, o] = sum over 128-wide K blocks kb, IN kb ORDER, of
//               dot128(E4M3 weights[o], E4M3 act codes[m]) * (as[m, kb] * 2^(ws[o/128, kb] - 127))
//
// (reference c/fp8.h:166-218: the scale product is formed first, one f32
// accumulator per output walks the blocks in order).  Each block dot is four
// `tcgen05.mma kind::f8f6f4` (K = 32) accumulating in tensor memory; the
// finished 128 x 32 block is read back (`tcgen05.ld`) by the epilogue warps and
// folded into f32 registers with that block's scales while the tensor core
// works on the next blocks in the other accumulators of a ring of four.  The fold order is
// therefore the reference's, for any K, with no split along K.
//
// Weights are read in the reference storage ([O, K] bytes, scales
// [O/128, K/128]) through a TMA tensor map: 128 x 128-byte tiles, 128-byte
// swizzle.  Algorithmic bytes per 128-row tile: 128*K + K/128.
//
// One CTA = one 128-row output tile for up to 32 activation rows (gate/up pair
// with fused SwiGLU optionally):
//   warp 4      TMA producer (weight tile(s) + 32 x 128 activation-code tile per stage)
//   warp 5      MMA issuer; owns the tensor-memory allocation
//   warps 0-3   per block: TMEM -> registers, fold with the scales; final epilogue
// mbarriers: full[s] / empty[s] for the shared-memory ring, acc_full[b] /
// acc_empty[b] for the ring of four accumulators.  Every wait is bounded; on expiry
// the CTA records a status word, drains and frees its tensor memory.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace apus {

__device__ int g_tc8_status = 0;         // first failure code (11..16) recorded by any CTA

namespace {

constexpr int T8_THREADS = 192;
constexpr int T8_N = 32;                 // activation rows per work item (MMA N)
constexpr int T8_A_BYTES = 128 * 128;    // one weight tile
constexpr int T8_B_BYTES = T8_N * 128;
constexpr int T8_MAX_NC = 128;           // K <= 16384

// Instruction descriptor, kind::f8f6f4: D = f32, A = B = E4M3, both K-major, M = 128, N = T8_N.
__device__ __forceinline__ uint32_t idesc_f8() {
    return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(T8_N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ float swiglu8(float gate, float up, float limit) {
    float g = bf16_round(gate), u = bf16_round(up);
    if (limit > 0.f) {
        u = fminf(fmaxf(u, -limit), limit);
        g = fminf(g, limit);
    }
    float sig = 1.0f / (1.0f + exp_rn(-g));
    return bf16_round(__fmul_rn(__fmul_rn(g, sig), u));
}

template <bool PAIR, int NS>
__global__ void __launch_bounds__(T8_THREADS, 2)
gemm_tc8_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                const __grid_constant__ CUtensorMap tm_x, const Tc8Args a) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int STAGE = T8_A_BYTES * (PAIR ? 2 : 1) + T8_B_BYTES;
    // ring of NACC accumulators (32 columns each; a pair uses two rings): the
    // MMA -> fold -> MMA round trip through the barriers takes longer than one
    // block's MMAs, so two accumulators leave the tensor core waiting
    constexpr int NACC = 4;
    constexpr int TMEM_COLS = PAIR ? 256 : 128;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)NS * STAGE);
    uint64_t *full = bars, *empty = bars + NS, *acc_full = bars + 2 * NS, *acc_empty = bars + 2 * NS + NACC;
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(bars + 2 * NS + 2 * NACC);
    volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem + 1);
    float *s_as = reinterpret_cast<float *>(s_tmem + 4);          // [NC][T8_N] activation scales
    const int K = a.K, O = a.O, NC = K >> 7, M = a.M;
    float *s_ws = s_as + (size_t)NC * T8_N;                        // [NC] weight tile scales (A), then (B)
    const int row0 = (int)blockIdx.y * T8_N;
    const int nrows = min(T8_N, M - row0);
    if (nrows <= 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile_row = (int)blockIdx.x * 128;
    // K chunk of this CTA: blocks [c0, c1) (the whole K unless the launch splits it, gridDim.z > 1)
    const int S = (int)gridDim.z, z = (int)blockIdx.z;
    const int c0 = (int)(((long long)NC * z) / S), c1 = (int)(((long long)NC * (z + 1)) / S);
    int *s_last = reinterpret_cast<int *>(s_tmem + 2);

    if (tid == 0) {
        for (int s = 0; s < NS; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < NACC; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
        *s_abort = 0;
        *s_last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // scales of this work item: as[kb][n] (0 for rows past the end) and the tile row of weight scales
    if (tid < 128) {
        for (int i = tid; i < NC * T8_N; i += 128) {
            const int kb = i / T8_N, n = i - kb * T8_N;
            s_as[i] = n < nrows ? a.ascales[(size_t)(row0 + n) * NC + kb] : 0.f;
        }
        const uint8_t *wsa = a.scales_a + (size_t)blockIdx.x * NC;
        for (int i = tid; i < NC; i += 128) {
            s_ws[i] = ue8m0_f32(wsa[i]);
            if (PAIR) s_ws[NC + i] = ue8m0_f32(a.scales_b[(size_t)blockIdx.x * NC + i]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;
    int fail = 0;

    if (warp == 4) {
        // ---- TMA producer ----------------------------------------------------------
        if (lane == 0) {
            for (int i = c0; i < c1 && !fail; i++) {
                const int it = i - c0, s = it % NS;
                const uint32_t ph = (uint32_t)(it / NS) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, s_abort)) { fail = 11; break; }
                uint8_t *st = smem + (size_t)s * STAGE;
                mbar_expect_tx(&full[s], STAGE);
                tma_load_2d(st, &tm_a, i * 128, tile_row, &full[s]);
                if (PAIR) tma_load_2d(st + T8_A_BYTES, &tm_b, i * 128, tile_row, &full[s]);
                tma_load_2d(st + T8_A_BYTES * (PAIR ? 2 : 1), &tm_x, i * 128, row0, &full[s]);
            }
        }
    } else if (warp == 5) {
        // ---- MMA issuer: block i accumulates into accumulator i % NACC -------------------
        if (lane == 0) {
            const uint32_t idesc = idesc_f8();
            for (int i = c0; i < c1 && !fail; i++) {
                const int it = i - c0, s = it % NS, b = it % NACC;
                const uint32_t ph = (uint32_t)(it / NS) & 1u, pb = (uint32_t)(it / NACC) & 1u;
                if (!mbar_wait(&acc_empty[b], pb ^ 1u, s_abort)) { fail = 12; break; }
                if (!mbar_wait(&full[s], ph, s_abort)) { fail = 13; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = smem_u32(smem + (size_t)s * STAGE);
                const uint64_t da = umma_desc_sw128(sa);
                const uint64_t db = umma_desc_sw128(sa + T8_A_BYTES);
                const uint64_t dx = umma_desc_sw128(sa + T8_A_BYTES * (PAIR ? 2 : 1));
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    umma_f8(tmem + b * 32, da + 2 * j, dx + 2 * j, idesc, j ? 1u : 0u);
                    if (PAIR) umma_f8(tmem + NACC * 32 + b * 32, db + 2 * j, dx + 2 * j, idesc, j ? 1u : 0u);
                }
                umma_commit(&empty[s]);                // the stage may be refilled once these MMAs retire
                umma_commit(&acc_full[b]);             // ... and the block is ready for the fold
            }
        }
    } else {
        // ---- fold (threads 0..127 = output rows of the tile) ------------------------------
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        float accA[T8_N], accB[PAIR ? T8_N : 1];
#pragma unroll
        for (int n = 0; n < T8_N; n++) accA[n] = 0.f;
        if (PAIR) {
#pragma unroll
            for (int n = 0; n < T8_N; n++) accB[n] = 0.f;
        }
        for (int i = c0; i < c1 && !fail; i++) {
            const int b = (i - c0) % NACC;
            const uint32_t pb = (uint32_t)((i - c0) / NACC) & 1u;
            if (!mbar_wait(&acc_full[b], pb, s_abort)) { fail = 14; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t d0[32], d1[32];
            tmem_ld32(tmem + lane_base + b * 32, d0);
            if (PAIR) tmem_ld32(tmem + lane_base + NACC * 32 + b * 32, d1);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&acc_empty[b]);                // the tensor core may overwrite this accumulator
            const float wsa = s_ws[i], wsb = PAIR ? s_ws[NC + i] : 0.f;
            const float4 *as4 = reinterpret_cast<const float4 *>(s_as + (size_t)i * T8_N);
            if (S > 1) {
                // K split: park this block's TERM dot * (as * ws) for every live row; the CTA that
                // finishes last adds all blocks' terms in block order -- the same values in the same
                // order as the single fold below, hence the same bits
                const int o = tile_row + tid;
                if (o < O) {
                    float *pa = a.part + ((size_t)i * M + row0) * O + o;
                    float *pb2 = a.part + ((size_t)(NC + i) * M + row0) * O + o;
                    for (int n = 0; n < nrows; n++) {
                        const float sv = s_as[(size_t)i * T8_N + n];
                        pa[(size_t)n * O] = __fmul_rn(__uint_as_float(d0[n]), __fmul_rn(sv, wsa));
                        if (PAIR) pb2[(size_t)n * O] = __fmul_rn(__uint_as_float(d1[n]), __fmul_rn(sv, wsb));
                    }
                }
                continue;
            }
#pragma unroll
            for (int q = 0; q < T8_N / 4; q++) {
                const float4 s4 = as4[q];
                const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const int n = 4 * q + r;
                    // the scale product is formed first, then one multiply and one add,
                    // each rounded (the reference is built without contraction)
                    accA[n] = __fadd_rn(accA[n], __fmul_rn(__uint_as_float(d0[n]), __fmul_rn(sv[r], wsa)));
                    if (PAIR)
                        accB[n] = __fadd_rn(accB[n], __fmul_rn(__uint_as_float(d1[n]), __fmul_rn(sv[r], wsb)));
                }
            }
        }
        if (!fail) {
            const int o = tile_row + tid;
            if (o < O && S == 1) {
#pragma unroll
                for (int n = 0; n < T8_N; n++) {
                    if (n >= nrows) break;
                    float v;
                    if (PAIR) v = swiglu8(accA[n], accB[n], a.limit);
                    else v = a.round_out ? bf16_round(accA[n]) : accA[n];
                    a.out[(size_t)(row0 + n) * O + o] = v;
                }
            } else if (o < O) {
                __threadfence();                       // this chunk's block terms are parked (fold loop above)
            }
        }
    }
    if (fail) {
        *s_abort = 1;
        atomicCAS(&g_tc8_status, 0, fail);
    }
    if (S > 1) {
        // the chunk that arrives last at this output tile adds every block's term in block order and finishes the rows
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && !*s_abort) {
            const int slot = (int)blockIdx.y * (int)gridDim.x + (int)blockIdx.x;
            const int prev = atomicAdd(&a.counters[slot], 1);
            if (prev == S - 1) { a.counters[slot] = 0; *s_last = 1; }     // left clean for the next launch
            __threadfence();
        }
        __syncthreads();
        const int o = tile_row + tid;
        if (*s_last && tid < 128 && o < O) {
            for (int n = 0; n < nrows; n++) {
                float va = 0.f, vb = 0.f;
                for (int c = 0; c < NC; c++) {
                    va = __fadd_rn(va, __ldcg(a.part + ((size_t)c * M + row0 + n) * O + o));
                    if (PAIR) vb = __fadd_rn(vb, __ldcg(a.part + ((size_t)(NC + c) * M + row0 + n) * O + o));
                }
                float v;
                if (PAIR) v = swiglu8(va, vb, a.limit);
                else v = a.round_out ? bf16_round(va) : va;
                a.out[(size_t)(row0 + n) * O + o] = v;
            }
        }
    }
    if (fail)       // give copies already issued to this CTA's shared memory time to land
        for (int i = 0; i < 2000; i++) __nanosleep(1000);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS)
                     : "memory");
}

// ---- many activation rows (prefill / large batches): 128 rows per CTA -----------------------
// Same structure with MMA N = 128: one weight tile is read once per 128
// activation rows instead of once per 32, two accumulators of 128 TMEM columns,
// and every fold thread keeps 128 running sums (its output row against the
// CTA's 128 activation rows).  The fold (3 CUDA-core operations per element per
// block: scale product, multiply, add -- the reference's order) costs more issue
// slots than the block's MMAs, so this kernel is bound by the FP32 pipe at about
// two thirds of the tensor peak; the per-block promotion is what keeps the
// result equal to the reference's block-ordered f32 fold.
constexpr int T8W_N = 128, T8W_NS = 5, T8W_NACC = 2;

__device__ __forceinline__ uint32_t idesc_f8_wide() {
    return (1u << 4) | ((uint32_t)(T8W_N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__global__ void __launch_bounds__(T8_THREADS, 1)
gemm_tc8_wide_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_x,
                     const Tc8Args a) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int B_BYTES = T8W_N * 128, STAGE = T8_A_BYTES + B_BYTES, NS = T8W_NS, NACC = T8W_NACC;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)NS * STAGE);
    uint64_t *full = bars, *empty = bars + NS, *acc_full = bars + 2 * NS, *acc_empty = bars + 2 * NS + NACC;
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(bars + 2 * NS + 2 * NACC);
    volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem + 1);
    float *s_as = reinterpret_cast<float *>(s_tmem + 4);          // [NC][128] activation scales
    const int K = a.K, O = a.O, NC = K >> 7, M = a.M;
    float *s_ws = s_as + (size_t)NC * T8W_N;                       // [NC] weight tile scales
    const int row0 = (int)blockIdx.y * T8W_N;
    const int nrows = min(T8W_N, M - row0);
    if (nrows <= 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile_row = (int)blockIdx.x * 128;

    if (tid == 0) {
        for (int s = 0; s < NS; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < NACC; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(s_tmem)), "r"(NACC * T8W_N) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid < 128) {
        for (int i = tid; i < NC * T8W_N; i += 128) {
            const int kb = i / T8W_N, n = i - kb * T8W_N;
            s_as[i] = n < nrows ? a.ascales[(size_t)(row0 + n) * NC + kb] : 0.f;
        }
        const uint8_t *wsa = a.scales_a + (size_t)blockIdx.x * NC;
        for (int i = tid; i < NC; i += 128) s_ws[i] = ue8m0_f32(wsa[i]);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;
    int fail = 0;

    if (warp == 4) {
        if (lane == 0) {
            for (int i = 0; i < NC && !fail; i++) {
                const int s = i % NS;
                const uint32_t ph = (uint32_t)(i / NS) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, s_abort)) { fail = 11; break; }
                uint8_t *st = smem + (size_t)s * STAGE;
                mbar_expect_tx(&full[s], STAGE);
                tma_load_2d(st, &tm_a, i * 128, tile_row, &full[s]);
                tma_load_2d(st + T8_A_BYTES, &tm_x, i * 128, row0, &full[s]);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            const uint32_t idesc = idesc_f8_wide();
            for (int i = 0; i < NC && !fail; i++) {
                const int s = i % NS, b = i % NACC;
                const uint32_t ph = (uint32_t)(i / NS) & 1u, pb = (uint32_t)(i / NACC) & 1u;
                if (!mbar_wait(&acc_empty[b], pb ^ 1u, s_abort)) { fail = 12; break; }
                if (!mbar_wait(&full[s], ph, s_abort)) { fail = 13; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = smem_u32(smem + (size_t)s * STAGE);
                const uint64_t da = umma_desc_sw128(sa), dx = umma_desc_sw128(sa + T8_A_BYTES);
#pragma unroll
                for (int j = 0; j < 4; j++) umma_f8(tmem + b * T8W_N, da + 2 * j, dx + 2 * j, idesc, j ? 1u : 0u);
                umma_commit(&empty[s]);
                umma_commit(&acc_full[b]);
            }
        }
    } else {
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        float acc[T8W_N];
#pragma unroll
        for (int n = 0; n < T8W_N; n++) acc[n] = 0.f;
        for (int i = 0; i < NC && !fail; i++) {
            const int b = i % NACC;
            const uint32_t pb = (uint32_t)(i / NACC) & 1u;
            if (!mbar_wait(&acc_full[b], pb, s_abort)) { fail = 14; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float ws = s_ws[i];
            const float4 *as4 = reinterpret_cast<const float4 *>(s_as + (size_t)i * T8W_N);
#pragma unroll
            for (int qd = 0; qd < T8W_N / 32; qd++) {
                uint32_t d[32];
                tmem_ld32(tmem + lane_base + b * T8W_N + qd * 32, d);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (qd == T8W_N / 32 - 1) {              // the accumulator has been read completely
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbar_arrive(&acc_empty[b]);
                }
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    const float4 s4 = as4[qd * 8 + q];
                    const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        const int n = qd * 32 + 4 * q + r;
                        acc[n] = __fadd_rn(acc[n], __fmul_rn(__uint_as_float(d[4 * q + r]), __fmul_rn(sv[r], ws)));
                    }
                }
            }
        }
        if (!fail) {
            const int o = tile_row + tid;
            if (o < O) {
#pragma unroll
                for (int n = 0; n < T8W_N; n++)
                    if (n < nrows) a.out[(size_t)(row0 + n) * O + o] = a.round_out ? bf16_round(acc[n]) : acc[n];
            }
        }
    }
    if (fail) {
        *s_abort = 1;
        atomicCAS(&g_tc8_status, 0, fail);
        for (int i = 0; i < 2000; i++) __nanosleep(1000);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NACC * T8W_N)
                     : "memory");
}

template <bool PAIR, int NS>
int launch_tc8(const Tc8Args &a, cudaStream_t st) {
    constexpr int STAGE = T8_A_BYTES * (PAIR ? 2 : 1) + T8_B_BYTES;
    const int NC = a.K >> 7;
    const size_t smem = (size_t)NS * STAGE + 1024 + 256 + (size_t)NC * T8_N * 4 + 2 * (size_t)NC * 4;
    auto kern = gemm_tc8_kernel<PAIR, NS>;
    if (ensure_dyn_smem((const void *)kern, 224 * 1024)) return 1;
    dim3 grid((unsigned)(a.O / 128), (unsigned)((a.M + T8_N - 1) / T8_N), (unsigned)(a.ksplit > 1 ? a.ksplit : 1));
    launch_k(kern, grid, T8_THREADS, smem, st, *reinterpret_cast<const CUtensorMap *>(a.map_a),
                                        *reinterpret_cast<const CUtensorMap *>(a.pair ? a.map_b : a.map_a),
                                        *reinterpret_cast<const CUtensorMap *>(a.map_x), a);
    APUS_LAUNCHED();
    return 0;
}

}  // namespace

// Tensor map over E4M3 weight codes [rows, K] bytes, 128 x 128 boxes.
int tc8_make_weight_map(void *out_map, const void *codes, long long rows, int K) {
    EncodeTiledFn fn = tc_encode_fn();
    APUS_REQUIRE(fn, "cuTensorMapEncodeTiled is not available from the driver");
    APUS_REQUIRE(K % 128 == 0 && ((uintptr_t)codes & 15) == 0, "tensor map: K=%d / base alignment", K);
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {128, 128}, estr[2] = {1, 1};
    CUresult r = fn(reinterpret_cast<CUtensorMap *>(out_map), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                    const_cast<void *>(codes), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    APUS_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(fp8 weights [%lld,%d]) failed: %d", rows, K, (int)r);
    return 0;
}

// a.map_x must be a map with 128-row boxes (tc8_make_act_map_wide)
int gemm_tc8_wide(const Tc8Args &a, cudaStream_t st) {
    APUS_REQUIRE(a.K % 128 == 0 && a.K <= 128 * 64 && a.O % 128 == 0 && !a.pair,
                 "gemm_tc8_wide: unsupported shape O=%d K=%d", a.O, a.K);
    if (a.M <= 0) return 0;
    const int NC = a.K >> 7;
    const size_t smem = (size_t)T8W_NS * (T8_A_BYTES + T8W_N * 128) + 1024 + 256 + (size_t)NC * T8W_N * 4 + (size_t)NC * 4;
    if (ensure_dyn_smem((const void *)gemm_tc8_wide_kernel, 224 * 1024)) return 1;
    dim3 grid((unsigned)(a.O / 128), (unsigned)((a.M + T8W_N - 1) / T8W_N));
    launch_k(gemm_tc8_wide_kernel, grid, T8_THREADS, smem, st, *reinterpret_cast<const CUtensorMap *>(a.map_a),
                                                         *reinterpret_cast<const CUtensorMap *>(a.map_x), a);
    APUS_LAUNCHED();
    return 0;
}

// Tensor map over E4M3 activation codes [rows, K] bytes with 128 x 128 boxes.
int tc8_make_act_map_wide(void *out_map, const void *codes, long long rows, int K) {
    return tc8_make_weight_map(out_map, codes, rows, K);
}

int gemm_tc8(const Tc8Args &a0, cudaStream_t st) {
    Tc8Args a = a0;
    APUS_REQUIRE(a.K % 128 == 0 && a.K <= 128 * T8_MAX_NC && a.O % 128 == 0,
                 "gemm_tc8: unsupported shape O=%d K=%d", a.O, a.K);
    if (a.M <= 0) return 0;
    long long ctas = (long long)(a.O / 128) * ((a.M + T8_N - 1) / T8_N);
    // A matrix with fewer output tiles than SMs streams on a few SMs only (each pulls ~25-45
    // GB/s): with few activation rows K is split over grid.z so that most SMs take part.  A chunk
    // does not fold: it parks every block's term dot * (as * ws); the CTA that finishes last adds
    // all terms in block order, which is the single in-order fold value for value -- the same
    // bits, whatever the split (so it needs no sum-order setting and a row's result does not
    // depend on the batch it is in).  Bounded to M <= 8 by the size of the parked terms.
    a.ksplit = 1;
    static const bool split_on = !(getenv("APUS_FP8_KSPLIT") && getenv("APUS_FP8_KSPLIT")[0] == '0');
    if (split_on && a.M <= 8 && ctas < 74) {
        const int NC = a.K >> 7;
        int S = (int)(148 / ctas);
        if (S > NC) S = NC;
        if (S > 32) S = 32;
        if (S > 1) {
            void *ws = nullptr;
            int *cnt = nullptr;
            if (stream_scratch(st, (size_t)NC * (a.pair ? 2 : 1) * a.M * a.O * 4, &ws, (size_t)ctas, &cnt)) return 1;
            a.ksplit = S; a.part = (float *)ws; a.counters = cnt;
            ctas *= S;
        }
    }
    // few CTAs: one CTA per SM with a deep ring, so that each CTA keeps ~200 KB of weight
    // tiles in flight; many CTAs: two per SM with a short ring
    if (a.pair) return ctas <= 148 ? launch_tc8<true, 5>(a, st) : launch_tc8<true, 3>(a, st);
    return ctas <= 148 ? launch_tc8<false, 10>(a, st) : launch_tc8<false, 4>(a, st);
}

int gemm_tc8_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc8_status, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v) {
        int z = 0;
        cudaMemcpyToSymbol(g_tc8_status, &z, sizeof(int));
    }
    return v;
}

}  // namespace apus
