// One-time re-tiling of quantised weights into tensor-core fragment order.
//
// The streaming GEMM kernels use mma.sync.m16n8k32 (E4M3 x E4M3 -> f32) with
// the weight matrix as the A operand: lane (g = lane/4, c = lane%4) of a warp
// holds, for a 16-row group and one 32-wide K block, eight K elements of row g
// and eight of row g+8.  The dot product does not care which K element sits in
// which MMA slot as long as both operands agree, so lane c is given the
// contiguous elements k = 8c .. 8c+7 of the block.  The tiled layouts below
// store exactly what each lane needs, contiguously, so that a warp's load is
// one coalesced 512-byte (MXFP4: two K blocks) or 512-byte (FP8: one K block)
// segment and no shared-memory staging or shuffling is needed.
//
// MXFP4 codes ("F4T"), 16 bytes per lane per pair of K blocks:
//   index ((rg * K/64 + kq) * 32 + lane) * 16, as four 32-bit words
//   [ (row g, blk 2kq), (row g+8, blk 2kq), (row g, blk 2kq+1), (row g+8, blk 2kq+1) ].
//   A word re-encodes eight E2M1 nibbles so that one byte-permute looks four of
//   them up as E4M3 bytes: nibble i keeps the 3-bit magnitude of element i in
//   its low bits; the spare top bit of each nibble carries a sign: bit 8j+7 is
//   the sign of element j (j<4), bit 8j+3 the sign of element 4+j.
// MXFP4 scales: ((rg * K/128 + kg) * 8 + g) * 8 bytes =
//   [ws(row g, blk 4kg..4kg+3), ws(row g+8, blk 4kg..4kg+3)].
// FP8 codes ("F8T"): ((rg * K/32 + kb) * 32 + lane) * 16 bytes =
//   [row g k0..3, row g+8 k0..3, row g k4..7, row g+8 k4..7], k0 = 32kb + 8c.
// FP8 scales stay in the reference layout [ceil(O/128), ceil(K/128)].
//
// Source formats: reference c/fp4.h:8-11 (low nibble = even K) and
// c/fp8.h:11-14.
#include "common.cuh"
#include "kernels.cuh"

namespace apus {

__global__ void repack_fp4_codes_kernel(const uint32_t *__restrict__ src,
                                        uint32_t *__restrict__ dst, int O, int K) {
    // one thread per output word
    size_t n_words = (size_t)O * K / 8;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_words) return;
    int j = (int)(i & 3);
    int lane = (int)((i >> 2) & 31);
    size_t t = i >> 7;
    int kq = (int)(t % (K / 64));
    int rg = (int)(t / (K / 64));
    int g = lane >> 2, c = lane & 3;
    int row = rg * 16 + g + ((j & 1) ? 8 : 0);
    int blk = 2 * kq + (j >> 1);
    uint32_t w = src[((size_t)row * (K / 2) + blk * 16 + 4 * c) >> 2];
    uint32_t mags = w & 0x77777777u;
    uint32_t sgn = w & 0x88888888u;
    uint32_t out = mags;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        out |= ((sgn >> (4 * e + 3)) & 1u) << (8 * e + 7);         // element e
        out |= ((sgn >> (4 * (4 + e) + 3)) & 1u) << (8 * e + 3);   // element 4+e
    }
    dst[i] = out;
}

__global__ void repack_fp4_scales_kernel(const uint8_t *__restrict__ src,
                                         uint8_t *__restrict__ dst, int O, int K,
                                         int *zero_flag) {
    size_t n = (size_t)O * K / 32;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int b = (int)(i & 3);
    int r = (int)((i >> 2) & 1);
    int g = (int)((i >> 3) & 7);
    size_t t = i >> 6;
    int kg = (int)(t % (K / 128));
    int rg = (int)(t / (K / 128));
    uint8_t v = src[(size_t)(rg * 16 + g + 8 * r) * (K / 32) + 4 * kg + b];
    if (v == 0 && zero_flag) atomicOr(zero_flag, 1);
    dst[i] = v;
}

__global__ void repack_fp8_kernel(const uint32_t *__restrict__ src,
                                  uint32_t *__restrict__ dst, int O, int K) {
    size_t n_words = (size_t)O * K / 4;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_words) return;
    int j = (int)(i & 3);
    int lane = (int)((i >> 2) & 31);
    size_t t = i >> 7;
    int kb = (int)(t % (K / 32));
    int rg = (int)(t / (K / 32));
    int g = lane >> 2, c = lane & 3;
    int row = rg * 16 + g + ((j & 1) ? 8 : 0);
    int k = kb * 32 + 8 * c + ((j >> 1) ? 4 : 0);
    dst[i] = src[((size_t)row * K + k) >> 2];
}

int repack_fp4(const uint8_t *packed, const uint8_t *scales, int O, int K,
               uint8_t *out_codes, uint8_t *out_scales, int *zero_scale_flag,
               cudaStream_t st) {
    APUS_REQUIRE(O % 16 == 0 && K % 128 == 0,
                 "MXFP4 weight [%d,%d]: O must be a multiple of 16 and K of 128", O, K);
    size_t nw = (size_t)O * K / 8;
    repack_fp4_codes_kernel<<<ceil_div(nw, 256), 256, 0, st>>>(
        (const uint32_t *)packed, (uint32_t *)out_codes, O, K);
    APUS_LAUNCHED();
    size_t ns = (size_t)O * K / 32;
    repack_fp4_scales_kernel<<<ceil_div(ns, 256), 256, 0, st>>>(
        scales, out_scales, O, K, zero_scale_flag);
    APUS_LAUNCHED();
    return 0;
}

int repack_fp8(const uint8_t *codes, int O, int K, uint8_t *out_codes,
               cudaStream_t st) {
    APUS_REQUIRE(O % 16 == 0 && K % 128 == 0,
                 "FP8 weight [%d,%d]: O must be a multiple of 16 and K of 128", O, K);
    size_t nw = (size_t)O * K / 4;
    repack_fp8_kernel<<<ceil_div(nw, 256), 256, 0, st>>>(
        (const uint32_t *)codes, (uint32_t *)out_codes, O, K);
    APUS_LAUNCHED();
    return 0;
}

}  // namespace apus
