// MoE glue kernels: router finish (sqrtsoftplus, bias, stable top-k / hash,
// weights), stable grouping of routings by expert, and the ordered combine.
#include "common.cuh"
#include "kernels.cuh"

namespace apus {

// ---- router ---------------------------------------------------------------------
//
// One CTA per token, one thread per expert (E <= 1024).  Reference
// c/moe.h:96-100, 352-367 (scores), c/attn.h:668-687 (stable top-k: strict
// greater-than, lowest index wins ties, descending order), c/moe.h:383-406
// (hash lookup; weights from the UNBIASED scores, summed in slot order,
// w = s / sum * route_scale).
__global__ void router_finish_kernel(const float *__restrict__ logits,
                                     const float *__restrict__ bias,
                                     const int64_t *__restrict__ tid2eid,
                                     const int64_t *__restrict__ ids, int E, int topk,
                                     float route_scale, float *__restrict__ sp_out,
                                     float *__restrict__ biased_out,
                                     int32_t *__restrict__ idx_out,
                                     float *__restrict__ wgt_out) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ float s_sp[];          // [E] unbiased scores
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ int s_sel[64];
    const int t = blockIdx.x, e = threadIdx.x;
    const int lane = e & 31, warp = e >> 5, nwarp = (blockDim.x + 31) >> 5;
    float sp = 0.f, key = -INFINITY;
    if (e < E) {
        float z = logits[(size_t)t * E + e];
        float soft = z > 20.0f ? z : log1p_rn(exp_rn(z));
        sp = sqrtf(soft);
        s_sp[e] = sp;
        if (sp_out) sp_out[(size_t)t * E + e] = sp;
        if (bias) {
            key = __fadd_rn(sp, bias[e]);
            if (biased_out) biased_out[(size_t)t * E + e] = key;
        }
    }
    __syncthreads();
    if (tid2eid) {
        if (e < topk) s_sel[e] = (int)tid2eid[ids[t] * topk + e];
    } else {
        bool used = (e >= E);
        for (int j = 0; j < topk; j++) {
            // argmax over unused entries; ties -> lowest index
            float v = used ? -INFINITY : key;
            int vi = used ? 0x7fffffff : e;
#pragma unroll
            for (int o = 16; o; o >>= 1) {
                float ov = __shfl_xor_sync(0xffffffffu, v, o);
                int oi = __shfl_xor_sync(0xffffffffu, vi, o);
                if (ov > v || (ov == v && oi < vi)) { v = ov; vi = oi; }
            }
            if (lane == 0) { s_val[warp] = v; s_idx[warp] = vi; }
            __syncthreads();
            if (warp == 0) {
                v = lane < nwarp ? s_val[lane] : -INFINITY;
                vi = lane < nwarp ? s_idx[lane] : 0x7fffffff;
#pragma unroll
                for (int o = 16; o; o >>= 1) {
                    float ov = __shfl_xor_sync(0xffffffffu, v, o);
                    int oi = __shfl_xor_sync(0xffffffffu, vi, o);
                    if (ov > v || (ov == v && oi < vi)) { v = ov; vi = oi; }
                }
                if (lane == 0) s_sel[j] = vi;
            }
            __syncthreads();
            if (s_sel[j] == e) used = true;
        }
    }
    __syncthreads();
    if (e == 0) {
        float sum = 0.f;
        for (int j = 0; j < topk; j++) sum = __fadd_rn(sum, s_sp[s_sel[j]]);
        for (int j = 0; j < topk; j++) {
            idx_out[(size_t)t * topk + j] = s_sel[j];
            wgt_out[(size_t)t * topk + j] =
                __fmul_rn(__fdiv_rn(s_sp[s_sel[j]], sum), route_scale);
        }
    }
}

int router_finish(const float *logits, const float *bias, const int64_t *tid2eid,
                  const int64_t *ids, int s, int E, int topk, float route_scale,
                  float *sp, float *biased, int32_t *idx, float *wgt,
                  cudaStream_t st) {
    APUS_REQUIRE(E <= 1024 && topk <= 64 && topk <= E, "router: E=%d topk=%d unsupported", E, topk);
    APUS_REQUIRE(bias || tid2eid, "router: neither a selection bias nor a hash table");
    if (s <= 0) return 0;
    int threads = ((E + 31) / 32) * 32;
    if (threads < 64) threads = 64;
    launch_k(router_finish_kernel, s, threads, E * sizeof(float), st, 
        logits, tid2eid ? nullptr : bias, tid2eid, ids, E, topk, route_scale, sp, biased,
        idx, wgt);
    APUS_LAUNCHED();
    return 0;
}

// ---- grouping -----------------------------------------------------------------------
//
// Stable counting sort of the routings by local expert (the reference's
// counting sort, c/moe.h:465-474) by one CTA, followed by the work-item table
// for the two GEMM passes: each expert's rows are cut into runs of at most
// `chunk` rows.  Routings whose expert is not local are skipped.  Rows of one
// expert keep their (token, slot) order: a routing's rank inside its expert is
// the number of earlier routings with the same expert id.
//   n <= GROUP_SMEM_N: ids staged in shared memory, one thread per routing
//     counts its predecessors; otherwise one warp per expert sweeps the list
//     with ballots.
#define GROUP_SMEM_N 4096
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int32_t *__restrict__ eid, const int32_t *__restrict__ row, int row_div,
                 int n, MoeSlab slab, int chunk, int *__restrict__ sorted_pos,
                 int *__restrict__ sorted_row, GemmGroup *__restrict__ g13,
                 GemmGroup *__restrict__ g2, int *__restrict__ n_groups, int max_groups,
                 TcGroup *__restrict__ t13, TcGroup *__restrict__ t2, int o13, int o2) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    __shared__ int s_cnt[1024], s_off[1024], s_goff[1024];
    __shared__ int s_eid[GROUP_SMEM_N];
    __shared__ int s_wsum[32], s_wgsum[32];
    const int nE = slab.e_hi - slab.e_lo;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const bool small = n <= GROUP_SMEM_N;
    for (int i = tid; i < nE; i += blockDim.x) s_cnt[i] = 0;
    __syncthreads();
    if (small) {
        for (int i = tid; i < n; i += blockDim.x) {
            int le = eid[i] - slab.e_lo;
            s_eid[i] = (le >= 0 && le < nE) ? le : -1;
            if (le >= 0 && le < nE) atomicAdd(&s_cnt[le], 1);
        }
    } else {
        for (int le = warp; le < nE; le += nwarp) {
            int cnt = 0;
            for (int base = 0; base < n; base += 32) {
                int i = base + lane;
                bool hit = i < n && eid[i] == slab.e_lo + le;
                cnt += __popc(__ballot_sync(0xffffffffu, hit));
            }
            if (lane == 0) s_cnt[le] = cnt;
        }
    }
    __syncthreads();
    // exclusive scans of the counts and of the per-expert work-item counts
    {
        int c = tid < nE ? s_cnt[tid] : 0;
        int g = (c + chunk - 1) / chunk;
        int ic = c, ig = g;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int tc = __shfl_up_sync(0xffffffffu, ic, o), tg = __shfl_up_sync(0xffffffffu, ig, o);
            if (lane >= o) { ic += tc; ig += tg; }
        }
        if (lane == 31) { s_wsum[warp] = ic; s_wgsum[warp] = ig; }
        __syncthreads();
        if (warp == 0) {
            int wc = s_wsum[lane], wg = s_wgsum[lane];
            int jc = wc, jg = wg;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int tc = __shfl_up_sync(0xffffffffu, jc, o), tg = __shfl_up_sync(0xffffffffu, jg, o);
                if (lane >= o) { jc += tc; jg += tg; }
            }
            s_wsum[lane] = jc - wc; s_wgsum[lane] = jg - wg;
            if (lane == 31) {
                n_groups[0] = jg < max_groups ? jg : max_groups;
                n_groups[1] = jc;                  // routings that are local
                n_groups[2] += n_groups[0];        // running total of work items (read by the timing interface)
            }
        }
        __syncthreads();
        if (tid < nE) { s_off[tid] = s_wsum[warp] + ic - c; s_goff[tid] = s_wgsum[warp] + ig - g; }
    }
    __syncthreads();
    if (small) {
        for (int i = tid; i < n; i += blockDim.x) {
            int le = s_eid[i];
            if (le < 0) continue;
            int rank = 0;
            for (int j = 0; j < i; j++) rank += (s_eid[j] == le);
            int p = s_off[le] + rank;
            sorted_pos[p] = i;
            sorted_row[p] = row ? row[i] : i / row_div;
        }
    } else {
        for (int le = warp; le < nE; le += nwarp) {
            int pos = s_off[le];
            for (int base = 0; base < n; base += 32) {
                int i = base + lane;
                bool hit = i < n && eid[i] == slab.e_lo + le;
                unsigned m = __ballot_sync(0xffffffffu, hit);
                if (hit) {
                    int p = pos + __popc(m & ((1u << lane) - 1u));
                    sorted_pos[p] = i;
                    sorted_row[p] = row ? row[i] : i / row_div;
                }
                pos += __popc(m);
            }
        }
    }
    for (int le = tid; le < nE; le += blockDim.x) {
        int cnt = s_cnt[le], gi = s_goff[le];
        for (int r = 0; r < cnt && gi < max_groups; r += chunk, gi++) {
            GemmGroup a, b;
            a.wa = slab.w1 + (size_t)le * slab.code_stride13;
            a.sa = slab.s1 + (size_t)le * slab.scale_stride13;
            a.wb = slab.w3 + (size_t)le * slab.code_stride13;
            a.sb = slab.s3 + (size_t)le * slab.scale_stride13;
            a.row0 = s_off[le] + r;
            a.nrows = min(chunk, cnt - r);
            b.wa = slab.w2 + (size_t)le * slab.code_stride2;
            b.sa = slab.s2 + (size_t)le * slab.scale_stride2;
            b.wb = nullptr; b.sb = nullptr;
            b.row0 = a.row0; b.nrows = a.nrows;
            g13[gi] = a; g2[gi] = b;
            if (t13) {
                TcGroup u = {le * o13, a.row0, a.nrows, 0}, v = {le * o2, a.row0, a.nrows, 0};
                t13[gi] = u; t2[gi] = v;
            }
        }
    }
}

int moe_group(const int32_t *rout_eid, const int32_t *rout_row, int row_div, int n_rout,
              const MoeSlab &slab, int chunk, int *sorted_pos, int *sorted_row,
              GemmGroup *g13, GemmGroup *g2, int *n_groups, int max_groups,
              cudaStream_t st, TcGroup *t13, TcGroup *t2, int o13, int o2) {
    APUS_REQUIRE(slab.e_hi - slab.e_lo <= 1024, "moe_group: more than 1024 local experts");
    APUS_REQUIRE(rout_row || row_div > 0, "moe_group: no row mapping");
    launch_k(moe_group_kernel, 1, 1024, 0, st, rout_eid, rout_row, row_div, n_rout, slab, chunk, sorted_pos,
                                         sorted_row, g13, g2, n_groups, max_groups, t13, t2, o13, o2);
    APUS_LAUNCHED();
    return 0;
}

// ---- combine ---------------------------------------------------------------------------
//
// y[t,i] = sum_j wgt[t,j] * eo[t*topk+j, i], j ascending, each step a rounded
// multiply then a rounded add (reference c/moe.h:148-158 is compiled without
// contraction); out = bf16(y + shared) (reference c/moe.h:584-585).
__global__ void moe_combine_kernel(const float *__restrict__ eo, const float *__restrict__ wgt,
                                   const float *__restrict__ shared, int topk, int dim,
                                   float *__restrict__ out, float *__restrict__ routed) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    int t = blockIdx.y;
    int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= dim) return;
    float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < topk; j++) {
        float w = wgt[(size_t)t * topk + j];
        float4 v = *reinterpret_cast<const float4 *>(eo + ((size_t)t * topk + j) * dim + i);
        y.x = __fadd_rn(y.x, __fmul_rn(w, v.x));
        y.y = __fadd_rn(y.y, __fmul_rn(w, v.y));
        y.z = __fadd_rn(y.z, __fmul_rn(w, v.z));
        y.w = __fadd_rn(y.w, __fmul_rn(w, v.w));
    }
    if (routed) *reinterpret_cast<float4 *>(routed + (size_t)t * dim + i) = y;
    if (out) {
        float4 s = shared ? *reinterpret_cast<const float4 *>(shared + (size_t)t * dim + i)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 o;
        o.x = bf16_round(__fadd_rn(y.x, s.x));
        o.y = bf16_round(__fadd_rn(y.y, s.y));
        o.z = bf16_round(__fadd_rn(y.z, s.z));
        o.w = bf16_round(__fadd_rn(y.w, s.w));
        *reinterpret_cast<float4 *>(out + (size_t)t * dim + i) = o;
    }
}

int moe_combine(const float *eo, const float *wgt, const float *shared, int s,
                int topk, int dim, float *out, float *routed, cudaStream_t st) {
    APUS_REQUIRE(dim % 4 == 0, "moe_combine: dim=%d", dim);
    if (s <= 0) return 0;
    dim3 grid((unsigned)ceil_div(dim / 4, 256), (unsigned)s);
    launch_k(moe_combine_kernel, grid, 256, 0, st, eo, wgt, shared, topk, dim, out, routed);
    APUS_LAUNCHED();
    return 0;
}

// ---- expert-parallel exchange helpers ---------------------------------------------------------------
// The slots of the fixed-shape exchange: routing p = t * topk + j goes to the rank
// that owns its expert, into that rank's block of `slots` row slots, in the order of
// p (a stable grouping by destination).  One CTA: a routing counts the earlier
// routings with its destination.  Unused slots keep expert id -1.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int32_t *__restrict__ idx, int n_rout, int per_rank, int world, int slots,
               int32_t *__restrict__ send_eids, int32_t *__restrict__ slot_of) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ int s_dest[];
    for (int i = threadIdx.x; i < world * slots; i += blockDim.x) send_eids[i] = -1;
    for (int p = threadIdx.x; p < n_rout; p += blockDim.x) s_dest[p] = idx[p] / per_rank;
    __syncthreads();
    for (int p = threadIdx.x; p < n_rout; p += blockDim.x) {
        const int d = s_dest[p];
        int before = 0;
        for (int q = 0; q < p; q++) before += s_dest[q] == d;
        const int slot = d * slots + before;
        slot_of[p] = slot;
        send_eids[slot] = idx[p];
    }
}
// gather == 0: dst[slot_of[p]] = src[p / topk]  (token rows into their slots)
// gather == 1: dst[p] = src[slot_of[p]]         (expert outputs back to (t, j) order)
__global__ void __launch_bounds__(256)
ep_rows_kernel(const float *__restrict__ src, int dim, const int32_t *__restrict__ slot_of, int topk, int gather,
               float *__restrict__ dst) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int p = blockIdx.x, slot = slot_of[p];
    const float4 *s4 = reinterpret_cast<const float4 *>(src + (size_t)(gather ? slot : p / topk) * dim);
    float4 *d4 = reinterpret_cast<float4 *>(dst + (size_t)(gather ? p : slot) * dim);
    for (int i = threadIdx.x; i < dim / 4; i += blockDim.x) d4[i] = s4[i];
}

// Quantised token rows as they travel between ranks: `dim` E4M3 codes followed by dim/128 f32
// scales (powers of two), EP_QROW(dim) bytes per row.
// pack: slot slot_of[p] of `packed` <- codes/scales of token row p / topk.
__global__ void __launch_bounds__(256)
ep_pack_q_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ scales, int dim,
                 const int32_t *__restrict__ slot_of, int topk, uint8_t *__restrict__ packed) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int p = blockIdx.x, row = p / topk, nab = dim >> 7;
    const size_t rb = (size_t)dim + (size_t)nab * 4;
    uint8_t *dst = packed + (size_t)slot_of[p] * rb;
    const uint4 *s4 = reinterpret_cast<const uint4 *>(codes + (size_t)row * dim);
    uint4 *d4 = reinterpret_cast<uint4 *>(dst);
    for (int i = threadIdx.x; i < dim / 16; i += blockDim.x) d4[i] = s4[i];
    float *ds = reinterpret_cast<float *>(dst + dim);
    for (int i = threadIdx.x; i < nab; i += blockDim.x) ds[i] = scales[(size_t)row * nab + i];
}
// unpack into sorted order: row p of codes/scales <- packed row sorted_row[p], for p < *n_dev
__global__ void __launch_bounds__(256)
ep_gather_q_kernel(const uint8_t *__restrict__ packed, int dim, const int *__restrict__ sorted_row,
                   const int *__restrict__ n_dev, uint8_t *__restrict__ codes, float *__restrict__ scales) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int p = blockIdx.x, nab = dim >> 7;
    if (p >= *n_dev) return;
    const size_t rb = (size_t)dim + (size_t)nab * 4;
    const uint8_t *src = packed + (size_t)sorted_row[p] * rb;
    const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
    uint4 *d4 = reinterpret_cast<uint4 *>(codes + (size_t)p * dim);
    for (int i = threadIdx.x; i < dim / 16; i += blockDim.x) d4[i] = s4[i];
    const float *ss = reinterpret_cast<const float *>(src + dim);
    for (int i = threadIdx.x; i < nab; i += blockDim.x) scales[(size_t)p * nab + i] = ss[i];
}
// expert outputs that came back as BF16 bits, to (t, j) order as f32: dst[p] = widen(src[slot_of[p]])
__global__ void __launch_bounds__(256)
ep_unpack_bf16_kernel(const uint16_t *__restrict__ src, int dim, const int32_t *__restrict__ slot_of,
                      float *__restrict__ dst) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int p = blockIdx.x;
    const uint2 *s2 = reinterpret_cast<const uint2 *>(src + (size_t)slot_of[p] * dim);
    float4 *d4 = reinterpret_cast<float4 *>(dst + (size_t)p * dim);
    for (int i = threadIdx.x; i < dim / 4; i += blockDim.x) {
        const uint2 v = s2[i];
        d4[i] = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u),
                            __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
    }
}
int ep_pack_q(const uint8_t *codes, const float *scales, int dim, const int32_t *slot_of, int n_rout, int topk,
              uint8_t *packed, cudaStream_t st) {
    if (n_rout <= 0) return 0;
    launch_k(ep_pack_q_kernel, n_rout, 256, 0, st, codes, scales, dim, slot_of, topk, packed);
    APUS_LAUNCHED();
    return 0;
}
int ep_gather_q(const uint8_t *packed, int dim, const int *sorted_row, const int *n_dev, int n_max, uint8_t *codes,
                float *scales, cudaStream_t st) {
    if (n_max <= 0) return 0;
    launch_k(ep_gather_q_kernel, n_max, 256, 0, st, packed, dim, sorted_row, n_dev, codes, scales);
    APUS_LAUNCHED();
    return 0;
}
int ep_unpack_bf16(const uint16_t *src, int dim, const int32_t *slot_of, int n_rout, float *dst, cudaStream_t st) {
    if (n_rout <= 0) return 0;
    launch_k(ep_unpack_bf16_kernel, n_rout, 256, 0, st, src, dim, slot_of, dst);
    APUS_LAUNCHED();
    return 0;
}

int ep_plan(const int32_t *idx, int n_rout, int per_rank, int world, int slots, int32_t *send_eids,
            int32_t *slot_of, cudaStream_t st) {
    launch_k(ep_plan_kernel, 1, 1024, (size_t)n_rout * sizeof(int), st, idx, n_rout, per_rank, world, slots, send_eids, slot_of);
    APUS_LAUNCHED();
    return 0;
}
int ep_rows(const float *src, int dim, const int32_t *slot_of, int n_rout, int topk, int gather, float *dst,
            cudaStream_t st) {
    launch_k(ep_rows_kernel, n_rout, 256, 0, st, src, dim, slot_of, topk, gather, dst);
    APUS_LAUNCHED();
    return 0;
}

}  // namespace apus
