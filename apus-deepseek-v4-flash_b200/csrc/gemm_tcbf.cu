// BF16 x BF16 -> f32 dense GEMV/GEMM on the 5th-generation tensor cores
// (tcgen05 kind::f16, BF16 operands): the vocabulary head (reference
// c/model.h:638-647), the grouped low-rank o-projection (c/attn.h:1692-1737) and
// every other dense linear whose weights are BF16 values (c/attn.h:621-666).
//
//   out[m, g*O + o] = sum_k x[m, g*xk + k] * w[g*O + o, k]        g = 0..batch-1
//
// BF16 x BF16 products are exact in f32; the tensor core adds them in its own
// order, so the result is the "tree order" class of apus_cuda_set_tree_ops: within
// ~1e-6 relative of the reference's sequential sum, not its bits.
//
// Weights are read where they lie ([rows, K] BF16, row-major) through a TMA
// tensor map: 128 rows x 64 elements (128-byte swizzled rows) per tile, each
// weight byte crosses HBM once.  Activations are BF16 copies [M, *] read the same
// way (32 rows per work item).  One CTA = one 128-row output tile x up to 32
// activation rows x one K chunk:
//   warp 4      TMA producer       warp 5      MMA issuer (owns the tensor memory)
//   warps 0-3   epilogue: TMEM -> registers -> out, or -> the K-split scratch
// With ksplit > 1 every chunk parks its partial sums in a scratch buffer and the
// CTA that finishes last (one counter per output tile) adds the chunks in chunk
// order and writes the result: matrices with few output tiles still stream on
// most SMs, and the sum stays deterministic.  Every wait is bounded.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace apus {

__device__ int g_tcbf_status = 0;        // first failure code (21..24) recorded by any CTA

namespace {

constexpr int TB_THREADS = 192;
constexpr int TB_N = 32;                 // activation rows per work item (MMA N)
constexpr int TB_KT = 64;                // K elements per tile (128 bytes)
constexpr int TB_A_BYTES = 128 * 128;
constexpr int TB_B_BYTES = TB_N * 128;
constexpr int TB_STAGE = TB_A_BYTES + TB_B_BYTES;

// Instruction descriptor, kind::f16: D = f32, A = B = BF16, both K-major, M = 128, N = TB_N.
__device__ __forceinline__ uint32_t idesc_bf16() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TB_N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

template <int NS>
__global__ void __launch_bounds__(TB_THREADS, 2)
gemm_tcbf_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const TcbfArgs a) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ uint8_t smem_raw[];
    __shared__ float s_amax[4][TB_N];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)NS * TB_STAGE);
    uint64_t *full = bars, *empty = bars + NS, *acc_full = bars + 2 * NS;
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(bars + 2 * NS + 1);
    volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem + 1);
    int *s_last = reinterpret_cast<int *>(s_tmem + 2);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // blockIdx.x = output tile over all problems, blockIdx.y = activation row group, blockIdx.z = K chunk
    const int tiles_per = a.O / 128;
    const int g = (int)blockIdx.x / tiles_per, tile = (int)blockIdx.x - g * tiles_per;
    const int row0 = (int)blockIdx.y * TB_N;
    const int nrows = min(TB_N, a.M - row0);
    const int NT = a.K / TB_KT;                         // K tiles of one problem
    const int S = (int)gridDim.z, z = (int)blockIdx.z;
    const int t0 = (int)(((long long)NT * z) / S), t1 = (int)(((long long)NT * (z + 1)) / S);
    const int w_row = g * a.O + tile * 128;             // first weight row of the tile
    const int xk0 = g * a.x_koff;                       // first activation column of the problem

    if (tid == 0) {
        for (int s = 0; s < NS; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        *s_abort = 0;
        *s_last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(s_tmem)), "r"(32) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;
    int fail = 0;

    if (warp == 4) {
        if (lane == 0) {
            for (int i = t0; i < t1 && !fail; i++) {
                const int it = i - t0, s = it % NS;
                const uint32_t ph = (uint32_t)(it / NS) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, s_abort)) { fail = 21; break; }
                uint8_t *st = smem + (size_t)s * TB_STAGE;
                mbar_expect_tx(&full[s], TB_STAGE);
                tma_load_2d(st, &tm_w, i * TB_KT, w_row, &full[s]);
                tma_load_2d(st + TB_A_BYTES, &tm_x, xk0 + i * TB_KT, row0, &full[s]);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            const uint32_t idesc = idesc_bf16();
            for (int i = t0; i < t1 && !fail; i++) {
                const int it = i - t0, s = it % NS;
                const uint32_t ph = (uint32_t)(it / NS) & 1u;
                if (!mbar_wait(&full[s], ph, s_abort)) { fail = 22; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = smem_u32(smem + (size_t)s * TB_STAGE);
                const uint64_t da = umma_desc_sw128(sa), dx = umma_desc_sw128(sa + TB_A_BYTES);
#pragma unroll
                for (int j = 0; j < 4; j++)                 // four K = 16 steps of 32 bytes inside the swizzled row
                    umma_bf16(tmem, da + 2 * j, dx + 2 * j, idesc, (it | j) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            if (!fail) umma_commit(acc_full);
        }
    } else {
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        if (!mbar_wait(acc_full, 0u, s_abort)) fail = 23;
        if (!fail) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t d[32];
            tmem_ld32(tmem + lane_base, d);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int o = tile * 128 + tid;                  // output column inside the problem
            const size_t col = (size_t)g * a.O + o;
            if (S == 1) {
#pragma unroll
                for (int n = 0; n < TB_N; n++)
                    if (n < nrows) {
                        const float v = __uint_as_float(d[n]);
                        a.out[(size_t)(row0 + n) * a.out_ld + col] = a.round_out ? bf16_round(v) : v;
                    }
            } else {
                // park this chunk's partial sums: part[z][row][col]
                const size_t ncol = (size_t)a.batch * a.O;
                float *part = a.part + ((size_t)z * a.M) * ncol;
#pragma unroll
                for (int n = 0; n < TB_N; n++)
                    if (n < nrows) part[(size_t)(row0 + n) * ncol + col] = __uint_as_float(d[n]);
                __threadfence();
            }
        }
    }
    if (fail) {
        *s_abort = 1;
        atomicCAS(&g_tcbf_status, 0, fail);
    }
    if (S > 1) {
        // the chunk that arrives last at this output tile adds the chunks in order
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && !*s_abort) {
            const int slot = (int)blockIdx.y * (int)gridDim.x + (int)blockIdx.x;
            const int prev = atomicAdd(&a.counters[slot], 1);
            if (prev == S - 1) { a.counters[slot] = 0; *s_last = 1; }     // leave the counter clean for the next launch
            __threadfence();
        }
        __syncthreads();
        if (*s_last && tid < 128) {
            const int o = tile * 128 + tid;
            const size_t col = (size_t)g * a.O + o, ncol = (size_t)a.batch * a.O;
            if (!a.q_out) {
                for (int n = 0; n < nrows; n++) {
                    float v = 0.f;
                    for (int c = 0; c < S; c++)
                        v = __fadd_rn(v, __ldcg(a.part + ((size_t)c * a.M + row0 + n) * ncol + col));
                    a.out[(size_t)(row0 + n) * a.out_ld + col] = a.round_out ? bf16_round(v) : v;
                }
            } else {
                // The finished tile holds 128 consecutive outputs of every row: one group of the activation
                // quantisation of the projection that reads them next (c/fp4.h:293-321).  Codes and scales
                // are made here -- amax over the four warps, power-of-two scale, hardware E4M3 conversion:
                // the arithmetic of act_quant_kernel -- instead of by a launch of their own.
                float vb[TB_N];
#pragma unroll
                for (int n = 0; n < TB_N; n++) {
                    if (n >= nrows) break;
                    float v = 0.f;
                    for (int c = 0; c < S; c++)
                        v = __fadd_rn(v, __ldcg(a.part + ((size_t)c * a.M + row0 + n) * ncol + col));
                    v = a.round_out ? bf16_round(v) : v;
                    a.out[(size_t)(row0 + n) * a.out_ld + col] = v;
                    vb[n] = bf16_round(v);
                    const float m = warp_max(fabsf(vb[n]));
                    if ((tid & 31) == 0) s_amax[tid >> 5][n] = m;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
                for (int n = 0; n < TB_N; n++) {
                    if (n >= nrows) break;
                    const float amax = fmaxf(fmaxf(fmaxf(s_amax[0][n], s_amax[1][n]), fmaxf(s_amax[2][n], s_amax[3][n])), 1e-4f);
                    const float sc = ceil_pow2(__fmul_rn(amax, 1.0f / 448.0f));
                    const float inv = __uint_as_float(0x7f000000u - __float_as_uint(sc));
                    a.q_out[(size_t)(row0 + n) * a.out_ld + col] = (uint8_t)(e4m3x2_from_f32(vb[n] * inv, 0.f) & 0xffu);
                    if (tid == 0) a.qs_out[((size_t)(row0 + n) * a.out_ld + col) >> 7] = sc;
                }
            }
        }
    }
    if (fail)
        for (int i = 0; i < 2000; i++) __nanosleep(1000);   // copies already issued to this CTA's shared memory land
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32) : "memory");
}

__global__ void f32_to_bf16_kernel(const float *x, uint16_t *y, long long n) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 v = *reinterpret_cast<const float4 *>(x + i);
        uint2 o;
        o.x = (uint32_t)bf16_bits(v.x) | ((uint32_t)bf16_bits(v.y) << 16);
        o.y = (uint32_t)bf16_bits(v.z) | ((uint32_t)bf16_bits(v.w) << 16);
        *reinterpret_cast<uint2 *>(y + i) = o;
    } else {
        for (long long k = i; k < n; k++) y[k] = bf16_bits(x[k]);
    }
}

int make_map_bf16(void *out_map, const void *base, long long rows, long long cols, int box_rows) {
    EncodeTiledFn fn = tc_encode_fn();
    APUS_REQUIRE(fn, "cuTensorMapEncodeTiled is not available from the driver");
    APUS_REQUIRE(cols % 8 == 0 && ((uintptr_t)base & 15) == 0, "BF16 tensor map: %lld columns / base alignment", cols);
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {TB_KT, (cuuint32_t)box_rows}, estr[2] = {1, 1};
    CUresult r = fn(reinterpret_cast<CUtensorMap *>(out_map), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    APUS_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(BF16 [%lld,%lld]) failed: %d", rows, cols, (int)r);
    return 0;
}

}  // namespace

int tcbf_make_weight_map(void *out_map, const void *w_bf16, long long rows, int K) {
    return make_map_bf16(out_map, w_bf16, rows, K, 128);
}
int tcbf_make_act_map(void *out_map, const void *x_bf16, long long rows, long long cols) {
    return make_map_bf16(out_map, x_bf16, rows, cols, TB_N);
}

int f32_to_bf16(const float *x, uint16_t *y, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    launch_k(f32_to_bf16_kernel, (unsigned)((n + 1023) / 1024), 256, 0, st, x, y, n);
    APUS_LAUNCHED();
    return 0;
}

// K chunks so that a launch with few output tiles still covers most SMs (each chunk at least 4 K tiles)
// The number of K chunks follows from the weight's shape alone: a row's sum is then cut the same
// way whatever the number of rows beside it, so one position and a chunk of positions agree bit for bit.
int tcbf_ksplit(int O, int K, int batch, int M) {
    (void)M;
    const long long ctas = (long long)(O / 128) * batch;
    const int nt = K / TB_KT;
    int s = (int)(148 / (ctas > 0 ? ctas : 1));
    if (s > nt / 4) s = nt / 4;
    if (s > 32) s = 32;
    return s < 1 ? 1 : s;
}

int gemm_tcbf(const TcbfArgs &a, cudaStream_t st) {
    APUS_REQUIRE(a.K % TB_KT == 0 && a.O % 128 == 0 && a.batch >= 1, "gemm_tcbf: unsupported shape O=%d K=%d", a.O, a.K);
    if (a.M <= 0) return 0;
    const int S = a.ksplit < 1 ? 1 : a.ksplit;
    APUS_REQUIRE(S == 1 || (a.part && a.counters), "gemm_tcbf: a K split needs the scratch buffers");
    APUS_REQUIRE(!a.q_out || (S > 1 && a.qs_out && a.out_ld % 128 == 0), "gemm_tcbf: codes are written by the K-split finish only");
    dim3 grid((unsigned)((a.O / 128) * a.batch), (unsigned)((a.M + TB_N - 1) / TB_N), (unsigned)S);
    const long long ctas = (long long)grid.x * grid.y * grid.z;
    const CUtensorMap *mw = reinterpret_cast<const CUtensorMap *>(a.map_w), *mx = reinterpret_cast<const CUtensorMap *>(a.map_x);
    if (ctas <= 148) {                                   // one CTA per SM: a deep ring hides the memory latency
        constexpr int NS = 10;
        if (ensure_dyn_smem((const void *)gemm_tcbf_kernel<NS>, NS * TB_STAGE + 2048)) return 1;
        launch_k(gemm_tcbf_kernel<NS>, grid, TB_THREADS, NS * TB_STAGE + 2048, st, *mw, *mx, a);
    } else {
        constexpr int NS = 5;
        if (ensure_dyn_smem((const void *)gemm_tcbf_kernel<NS>, NS * TB_STAGE + 2048)) return 1;
        launch_k(gemm_tcbf_kernel<NS>, grid, TB_THREADS, NS * TB_STAGE + 2048, st, *mw, *mx, a);
    }
    APUS_LAUNCHED();
    return 0;
}

int gemm_tcbf_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tcbf_status, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v) {
        int z = 0;
        cudaMemcpyToSymbol(g_tcbf_status, &z, sizeof(int));
    }
    return v;
}

}  // namespace apus
