// MXFP4 expert GEMV/GEMM on the 5th-generation tensor cores (tcgen05).
//
// out[n, o] = sum over 32-wide K blocks of (dot32(E4M3 act codes, E2M1 weights)
//             * act_scale[n, kb/4]) * 2^(wscale[o, kb] - 127)
// (reference c/fp4.h:367-395) computed by `tcgen05.mma kind::mxf8f6f4
// .block_scale`: the hardware expands the E2M1 codes, applies both UE8M0 scale
// factors per 32-element block and accumulates in f32 in tensor memory, so no
// CUDA-core work is spent per weight element.  Activation scales are powers
// of two, so their f32 exponent byte is the UE8M0 scale.  The result differs
// from the reference's sequential f32 fold only by summation order.
//
// Weights are read in the REFERENCE storage (packed nibbles [O, K/2], scales
// [O, K/32]): a TMA tensor map of type 16U4_ALIGN16B unpacks 128x128-element
// tiles into 128-byte swizzled shared-memory rows, 4.25 bits per weight cross
// HBM.  Algorithmic bytes per 128-row tile and matrix: 128*K/2 + 128*K/32.
//
// One CTA = one 128-row output tile of one work item (a gate/up pair or a
// single matrix) for up to 32 activation rows:
//   warp 4      TMA producer: per 128-wide K chunk the weight tile(s) and the
//               32 x 128 activation-code tile into a ring of shared-memory stages;
//   warps 0-3   scale-factor loaders: per chunk, four UE8M0 bytes per weight row
//               and per activation row, written to tensor memory in the layout
//               the MMA expects (row 32*j + l in lane l, column j, replicated
//               in the four 32-lane quadrants); afterwards the epilogue
//               (TMEM -> registers -> BF16 round / SwiGLU -> global);
//   warp 5      MMA issuer: four K=32 MMAs per chunk and matrix, scale-factor
//               byte selected per MMA through the instruction descriptor.
// mbarriers: full[s] (TMA bytes landed), sf_full[s] (scale factors stored),
// empty[s] (MMAs of the stage retired, via tcgen05.commit), done.
// Every wait is bounded; on expiry the CTA records a status word, drains and
// frees its tensor memory instead of hanging.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace apus {

__device__ int g_tc_status = 0;

namespace {

constexpr int TC_THREADS = 192;
constexpr int TC_N = 32;                 // activation rows per work item (MMA N)
constexpr int TC_A_BYTES = 128 * 128;    // one weight tile in shared memory
constexpr int TC_B_BYTES = TC_N * 128;
constexpr int TC_TMEM_COLS = 128;
constexpr int TC_COL_D0 = 0, TC_COL_D1 = 32, TC_COL_SF = 64, TC_SF_STRIDE = 12;
// Instruction descriptor, kind::mxf8f6f4 block-scaled: A = E2M1, B = E4M3, both
// K-major, UE8M0 scales, M = 128, N = TC_N; sf ids pick the scale byte.
__device__ __forceinline__ uint32_t umma_idesc(uint32_t a_sf, uint32_t b_sf) {
    return (b_sf << 4) | (5u << 7) | (0u << 10) | ((uint32_t)(TC_N >> 3) << 17) | (1u << 23) |
           ((uint32_t)(128 >> 4) << 24) | (a_sf << 29);
}
__device__ __forceinline__ void umma_mxf8f6f4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                              uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
__device__ __forceinline__ float swiglu_tc(float gate, float up, float limit) {
    float g = bf16_round(gate), u = bf16_round(up);
    if (limit > 0.f) {
        u = fminf(fmaxf(u, -limit), limit);
        g = fminf(g, limit);
    }
    float sig = 1.0f / (1.0f + exp_rn(-g));
    return bf16_round(__fmul_rn(__fmul_rn(g, sig), u));
}

template <bool PAIR, int NS>
__global__ void __launch_bounds__(TC_THREADS, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ CUtensorMap tm_x, const TcArgs a) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int STAGE = TC_A_BYTES * (PAIR ? 2 : 1) + TC_B_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)NS * STAGE);
    uint64_t *full = bars, *empty = bars + NS, *sf_full = bars + 2 * NS, *done = bars + 3 * NS;
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(bars + 3 * NS + 1);
    volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem + 1);
    int *s_last = reinterpret_cast<int *>(s_tmem + 2);

    const int n_groups = a.n_groups_dev ? *a.n_groups_dev : a.n_groups;
    if ((int)blockIdx.y >= n_groups) return;
    const TcGroup grp = a.groups[blockIdx.y];
    const int nrows = grp.nrows, row0 = grp.row0;
    if (nrows <= 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = a.K, O = a.O, NC = K >> 7;
    const int tile_row = grp.a_row + (int)blockIdx.x * 128;     // row in the weight slab
    // K chunk of this CTA (gridDim.z > 1: a launch with few work items splits K so that most SMs
    // stream): 128-wide chunks [c0, c1), whole batches of four (the scale loaders fetch 16 bytes)
    const int S = (int)gridDim.z, z = (int)blockIdx.z;
    const int b0 = (int)(((long long)(NC >> 2) * z) / S), b1 = (int)(((long long)(NC >> 2) * (z + 1)) / S);
    const int c0 = 4 * b0, c1 = 4 * b1;

    if (tid == 0) {
        for (int s = 0; s < NS; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&sf_full[s], 128); }
        mbar_init(done, 1);
        *s_abort = 0;
        *s_last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {                                   // tensor-memory allocation (one warp)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(s_tmem)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;
    int fail = 0;

    if (warp == 4) {
        // ---- TMA producer --------------------------------------------------------
        if (lane == 0) {
            for (int i = c0; i < c1 && !fail; i++) {
                const int s = (i - c0) % NS;
                const uint32_t ph = (uint32_t)((i - c0) / NS) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, s_abort)) { fail = 1; break; }
                uint8_t *st = smem + (size_t)s * STAGE;
                // the transaction count of a packed 4-bit tile is its global-memory size
                // (64 B per row), not the 128 B per row it occupies in shared memory
                mbar_expect_tx(&full[s], a.tx_bytes ? a.tx_bytes
                                                    : (TC_A_BYTES / 2) * (PAIR ? 2 : 1) + TC_B_BYTES);
                tma_load_2d(st, &tm_a, i * 128, tile_row, &full[s]);
                if (PAIR) tma_load_2d(st + TC_A_BYTES, &tm_b, i * 128, tile_row, &full[s]);
                tma_load_2d(st + TC_A_BYTES * (PAIR ? 2 : 1), &tm_x, i * 128, row0, &full[s]);
            }
        }
    } else if (warp == 5) {
        // ---- MMA issuer -------------------------------------------------------------
        if (lane == 0) {
            for (int i = c0; i < c1 && !fail; i++) {
                const int s = (i - c0) % NS;
                const uint32_t ph = (uint32_t)((i - c0) / NS) & 1u;
                if (!mbar_wait(&full[s], ph, s_abort)) { fail = 2; break; }
                if (!mbar_wait(&sf_full[s], ph, s_abort)) { fail = 5; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = smem_u32(smem + (size_t)s * STAGE);
                const uint64_t da = umma_desc_sw128(sa);
                const uint64_t db = umma_desc_sw128(sa + TC_A_BYTES);
                const uint64_t dx = umma_desc_sw128(sa + TC_A_BYTES * (PAIR ? 2 : 1));
                const uint32_t sf = tmem + TC_COL_SF + s * TC_SF_STRIDE;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t idesc = umma_idesc(j, j);
                    const uint32_t acc = ((i - c0) | j) ? 1u : 0u;
                    umma_mxf8f6f4(tmem + TC_COL_D0, da + 2 * j, dx + 2 * j, idesc, sf, sf + 8, acc);
                    if (PAIR) umma_mxf8f6f4(tmem + TC_COL_D1, db + 2 * j, dx + 2 * j, idesc, sf + 4, sf + 8, acc);
                }
                umma_commit(&empty[s]);
            }
            if (!fail) umma_commit(done);
        }
    } else {
        // ---- scale-factor loaders (threads 0..127) -----------------------------------
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const int nbk = K >> 5;                        // scale bytes per weight row
        const uint8_t *sA = a.scales_a + (size_t)tile_row * nbk;
        const uint8_t *sB = PAIR ? a.scales_b + (size_t)tile_row * nbk : nullptr;
        const float *xs = a.ascales + (size_t)(row0 + lane) * NC;
        const bool xrow_ok = lane < nrows;
        // scale bytes are fetched four chunks (16 bytes per weight row) at a time and
        // one batch ahead of their use, so that no global-memory latency sits
        // between two stages
        uint4 ca[4], cb[4], na[4], nb[4];
        float4 cx = make_float4(0.f, 0.f, 0.f, 0.f), nx = cx;
        auto load_batch = [&](int i4, uint4 (&ya)[4], uint4 (&yb)[4], float4 &yx) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                ya[j] = __ldg(reinterpret_cast<const uint4 *>(sA + (size_t)(32 * j + lane) * nbk) + i4);
                if (PAIR) yb[j] = __ldg(reinterpret_cast<const uint4 *>(sB + (size_t)(32 * j + lane) * nbk) + i4);
            }
            if (xrow_ok) yx = __ldg(reinterpret_cast<const float4 *>(xs) + i4);
        };
        auto comp = [](const uint4 &v, int c) { return c == 0 ? v.x : c == 1 ? v.y : c == 2 ? v.z : v.w; };
        auto compf = [](const float4 &v, int c) { return c == 0 ? v.x : c == 1 ? v.y : c == 2 ? v.z : v.w; };
        // K is a multiple of 512 on this path: batches [b0, b1) of four chunks
        load_batch(b0, ca, cb, cx);
        for (int i4 = b0; i4 < b1 && !fail; i4++) {
            if (i4 + 1 < b1) load_batch(i4 + 1, na, nb, nx);
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                const int i = i4 * 4 + cc;
                const int s = (i - c0) % NS;
                const uint32_t ph = (uint32_t)((i - c0) / NS) & 1u;
                uint32_t xb = 0;
                if (xrow_ok) xb = ((__float_as_uint(compf(cx, cc)) >> 23) & 0xffu) * 0x01010101u;
                if (!mbar_wait(&empty[s], ph ^ 1u, s_abort)) { fail = 3; break; }
                const uint32_t sf = tmem + lane_base + TC_COL_SF + s * TC_SF_STRIDE;
                tmem_st4(sf, comp(ca[0], cc), comp(ca[1], cc), comp(ca[2], cc), comp(ca[3], cc));
                if (PAIR) tmem_st4(sf + 4, comp(cb[0], cc), comp(cb[1], cc), comp(cb[2], cc), comp(cb[3], cc));
                tmem_st1(sf + 8, xb);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(&sf_full[s]);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) { ca[j] = na[j]; if (PAIR) cb[j] = nb[j]; }
            cx = nx;
        }
        // ---- epilogue ------------------------------------------------------------------
        if (!fail && !mbar_wait(done, 0, s_abort)) fail = 4;
        if (!fail) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t d0[32], d1[32];
            tmem_ld32(tmem + lane_base + TC_COL_D0, d0);
            if (PAIR) tmem_ld32(tmem + lane_base + TC_COL_D1, d1);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int o = (int)blockIdx.x * 128 + tid;
            if (PAIR && S == 1 && a.q_out) {
                // The SwiGLU outputs feed the down projection, whose activation quantisation works on 128
                // consecutive elements of a row (c/fp4.h:293-321): exactly this tile's 128 outputs of
                // one token.  Quantise here (amax over the four epilogue warps, power-of-two scale,
                // hardware E4M3 conversion -- the arithmetic of act_quant_kernel, hence its bits) and
                // write codes + scales instead of the f32 values and a separate launch.
                float *s_amax = reinterpret_cast<float *>(smem);       // [4][TC_N]: the stages are idle by now
                float hv[TC_N];
#pragma unroll
                for (int n = 0; n < TC_N; n++) {
                    if (n >= nrows) break;                 // a work item at decode sizes holds one to three rows
                    hv[n] = swiglu_tc(__uint_as_float(d0[n]), __uint_as_float(d1[n]), a.limit);
                    const float m = warp_max(fabsf(hv[n]));
                    if (lane == 0) s_amax[warp * TC_N + n] = m;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int nab = O >> 7;
#pragma unroll
                for (int n = 0; n < TC_N; n++) {
                    if (n >= nrows) break;
                    float amax = fmaxf(fmaxf(s_amax[n], s_amax[TC_N + n]), fmaxf(s_amax[2 * TC_N + n], s_amax[3 * TC_N + n]));
                    amax = fmaxf(amax, 1e-4f);
                    const float sc = ceil_pow2(__fmul_rn(amax, 1.0f / 448.0f));
                    const float inv = __uint_as_float(0x7f000000u - __float_as_uint(sc));
                    a.q_out[(size_t)(row0 + n) * O + o] = (uint8_t)(e4m3x2_from_f32(hv[n] * inv, 0.f) & 0xffu);
                    if (tid == 0) a.qs_out[(size_t)(row0 + n) * nab + blockIdx.x] = sc;
                }
            } else if (o < O && S == 1) {
#pragma unroll
                for (int n = 0; n < TC_N; n++) {
                    if (n >= nrows) break;
                    const int dst = a.orow ? a.orow[row0 + n] : row0 + n;
                    float v;
                    if (PAIR) v = swiglu_tc(__uint_as_float(d0[n]), __uint_as_float(d1[n]), a.limit);
                    else v = a.round_out ? bf16_round(__uint_as_float(d0[n])) : __uint_as_float(d0[n]);
                    a.out[(size_t)dst * O + o] = v;
                }
            } else if (o < O) {
                // park this chunk's sums: part[(matrix, chunk)][sorted row][o]
                float *pa = a.part + ((size_t)z * a.total_rows) * O;
                float *pb = a.part + ((size_t)(S + z) * a.total_rows) * O;
#pragma unroll
                for (int n = 0; n < TC_N; n++) {
                    if (n >= nrows) break;
                    pa[(size_t)(row0 + n) * O + o] = __uint_as_float(d0[n]);
                    if (PAIR) pb[(size_t)(row0 + n) * O + o] = __uint_as_float(d1[n]);
                }
                __threadfence();
            }
        }
    }
    if (fail) {
        *s_abort = 1;
        atomicCAS(&g_tc_status, 0, fail);
    }
    if (S > 1) {
        // the chunk that arrives last at this (tile, work item) adds the chunks in order and finishes the rows
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && !*s_abort) {
            const int slot = (int)blockIdx.y * (int)gridDim.x + (int)blockIdx.x;
            const int prev = atomicAdd(&a.counters[slot], 1);
            if (prev == S - 1) { a.counters[slot] = 0; *s_last = 1; }
            __threadfence();
        }
        __syncthreads();
        const int o = (int)blockIdx.x * 128 + tid;
        if (*s_last && tid < 128 && o < O) {
            for (int n = 0; n < nrows; n++) {
                float va = 0.f, vb = 0.f;
                for (int c = 0; c < S; c++) {
                    va = __fadd_rn(va, __ldcg(a.part + ((size_t)c * a.total_rows + row0 + n) * O + o));
                    if (PAIR) vb = __fadd_rn(vb, __ldcg(a.part + ((size_t)(S + c) * a.total_rows + row0 + n) * O + o));
                }
                const int dst = a.orow ? a.orow[row0 + n] : row0 + n;
                float v;
                if (PAIR) v = swiglu_tc(va, vb, a.limit);
                else v = a.round_out ? bf16_round(va) : va;
                a.out[(size_t)dst * O + o] = v;
            }
        }
    }
    if (fail)       // give copies already issued to this CTA's shared memory time to land
        for (int i = 0; i < 2000; i++) __nanosleep(1000);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS)
                     : "memory");
}

}  // namespace

EncodeTiledFn tc_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Tensor map over packed E2M1 codes [rows, K/2] (K elements per row), 128x128 boxes.
int tc_make_weight_map(void *out_map, const void *codes, long long rows, int K) {
    EncodeTiledFn fn = tc_encode_fn();
    APUS_REQUIRE(fn, "cuTensorMapEncodeTiled is not available from the driver");
    APUS_REQUIRE(K % 128 == 0 && ((uintptr_t)codes & 31) == 0, "tensor map: K=%d / base alignment", K);
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
    cuuint32_t box[2] = {128, 128}, estr[2] = {1, 1};
    CUresult r = fn(reinterpret_cast<CUtensorMap *>(out_map), CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2,
                    const_cast<void *>(codes), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    APUS_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(weights [%lld,%d]) failed: %d", rows, K, (int)r);
    return 0;
}

// Tensor map over E4M3 activation codes [rows, K] bytes, 128 x 32 boxes.
int tc_make_act_map(void *out_map, const void *codes, long long rows, int K) {
    EncodeTiledFn fn = tc_encode_fn();
    APUS_REQUIRE(fn, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {128, TC_N}, estr[2] = {1, 1};
    CUresult r = fn(reinterpret_cast<CUtensorMap *>(out_map), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                    const_cast<void *>(codes), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    APUS_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(acts [%lld,%d]) failed: %d", rows, K, (int)r);
    return 0;
}

template <bool PAIR, int NS>
static int launch_tc(const TcArgs &a, cudaStream_t st) {
    constexpr int STAGE = TC_A_BYTES * (PAIR ? 2 : 1) + TC_B_BYTES;
    const size_t smem = (size_t)NS * STAGE + 1024 + 256;
    auto kern = gemm_tc_kernel<PAIR, NS>;
    if (ensure_dyn_smem((const void *)kern, smem)) return 1;
    dim3 grid((unsigned)(a.O / 128), (unsigned)a.n_groups, (unsigned)(a.ksplit > 1 ? a.ksplit : 1));
    launch_k(kern, grid, TC_THREADS, smem, st, *reinterpret_cast<const CUtensorMap *>(a.map_a),
                                        *reinterpret_cast<const CUtensorMap *>(a.pair ? a.map_b : a.map_a),
                                        *reinterpret_cast<const CUtensorMap *>(a.map_x), a);
    APUS_LAUNCHED();
    return 0;
}

int gemm_tc(const TcArgs &a0, cudaStream_t st) {
    TcArgs a = a0;
    APUS_REQUIRE(a.K % 512 == 0 && a.O % 128 == 0, "gemm_tc: unsupported shape O=%d K=%d", a.O, a.K);
    if (a.n_groups <= 0) return 0;
    // Optional K split of the gate/up pair (APUS_TC_KSPLIT=2 or 4; off by default): grid.z chunks
    // whose sums the CTA that finishes last adds in chunk order.  It depends on the shape only,
    // never on the number of work items, so a token's result does not depend on the batch it is in
    // or on how many experts the rank holds.  Measured on the six-layer slice it buys nothing at
    // batch 1 (2.31 vs 2.32 ms per step: the launch is bound by the per-chunk hand-offs of a CTA,
    // not by the number of CTAs) and costs 8 % at batch 32, hence off.
    a.ksplit = 1;
    const long long ctas = (long long)(a.O / 128) * a.n_groups;
    static const int want = getenv("APUS_TC_KSPLIT") ? atoi(getenv("APUS_TC_KSPLIT")) : 1;
    if (a.total_rows > 0 && a.pair && want > 1) {
        const int nb4 = a.K >> 9;
        int S = want;
        while (S > 1 && (nb4 % S || S > nb4)) S--;
        if (S > 1) {
            void *ws = nullptr;
            int *cnt = nullptr;
            if (stream_scratch(st, (size_t)S * (a.pair ? 2 : 1) * a.total_rows * a.O * 4, &ws, (size_t)ctas, &cnt)) return 1;
            a.ksplit = S; a.part = (float *)ws; a.counters = cnt;
        }
    }
    static const int pns = getenv("APUS_TC_PAIR_NS") ? atoi(getenv("APUS_TC_PAIR_NS")) : 3;
    if (a.pair) return pns == 2 ? launch_tc<true, 2>(a, st) : launch_tc<true, 3>(a, st);
    // single matrix (the down projection, K = 2048: 16 chunks per CTA): the K loop is short, so the
    // fill and drain of a CTA's ring weigh as much as its steady state; a shallower ring lets more
    // CTAs share an SM (shared memory is what bounds them) and overlap each other's ends
    static const int ns = getenv("APUS_TC_DOWN_NS") ? atoi(getenv("APUS_TC_DOWN_NS")) : 3;
    if (ns == 2) return launch_tc<false, 2>(a, st);
    if (ns == 3) return launch_tc<false, 3>(a, st);
    return launch_tc<false, 5>(a, st);
}

// Status word of the bounded waits (0 = no failure since the last reset).
int gemm_tc_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v) {
        int z = 0;
        cudaMemcpyToSymbol(g_tc_status, &z, sizeof(int));
    }
    const int v8 = gemm_tc8_status(reset);          // the FP8 kernel keeps its own word (codes 11..15)
    const int vb = gemm_tcbf_status(reset);         // and the BF16 kernel (codes 21..23)
    return v ? v : (v8 ? v8 : vb);
}

}  // namespace apus
