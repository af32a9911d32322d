/*
 * apus_synth.h — counter-based synthetic tensors for random-init models.
 *
 * Every element of every tensor is a pure function of (key, element index):
 * a splitmix64 hash, then integer or exactly-rounded f32 arithmetic only (no
 * libm), so a CUDA kernel and plain host code produce the same bits.  A model
 * of any size can therefore be generated in HBM without crossing PCIe, and a
 * CPU checker can regenerate any tensor of it on demand and run the reference
 * on identical weights.  No counterpart in the reference (its tests draw their
 * fixtures from numpy, tests/m3/gen_golden.py).
 *
 * Both fill functions live in libapus_b200.so; the host one needs no GPU.
 */
#ifndef APUS_SYNTH_H
#define APUS_SYNTH_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    /* u8: every byte uniform over 0..255 (two uniform E2M1 nibbles) */
    APUS_SYNTH_U8 = 0,
    /* u8: uniform over [a, b] (integers; UE8M0 scale bytes) */
    APUS_SYNTH_U8_RANGE = 1,
    /* f32: a + b * z, z ~ approximately N(0,1) (sum of four 16-bit uniforms) */
    APUS_SYNTH_F32 = 2,
    /* f32 carrying BF16 values: the same, rounded to BF16 (RNE) */
    APUS_SYNTH_F32_BF16 = 3,
    /* u16 BF16 bits of a + b * z */
    APUS_SYNTH_BF16 = 4,
    /* u8 E4M3 codes of (a + b * z), RNE, saturating at +-448 */
    APUS_SYNTH_E4M3 = 5,
    /* i64: uniform over [0, a) */
    APUS_SYNTH_I64_MOD = 6,
    /* i64 rows of k = (int)b distinct values in [0, a): element i belongs to
     * row i / k (hash-routing tables, c/moe.h:42); n must be a multiple of k */
    APUS_SYNTH_I64_SUBSET = 7
} ApusSynthKind;

/* The key of one tensor: a hash of (seed, layer, tensor id, expert). */
uint64_t apus_synth_key(uint64_t seed, uint32_t layer, uint32_t tensor, uint32_t expert);

/* Fill n elements of `dst` (host memory). threads <= 0: all cores (at most 32). */
int apus_synth_fill_host(void *dst, int kind, uint64_t n, uint64_t key, double a, double b,
                         int threads);
/* The same into device memory, asynchronously on `stream` (a cudaStream_t). */
int apus_synth_fill_dev(void *dst, int kind, uint64_t n, uint64_t key, double a, double b,
                        void *stream);

/* n_seg consecutive tensors of n elements each (an expert-major slab) in ONE launch: segment s
 * is filled with the key apus_synth_key(seed, layer, tensor, first_expert + s), i.e. with the
 * bytes n_seg separate fills would write.  Kinds U8 .. E4M3. */
int apus_synth_fill_slab_dev(void *dst, int kind, uint64_t n, uint32_t n_seg, uint64_t seed,
                             uint32_t layer, uint32_t tensor, uint32_t first_expert, double a,
                             double b, void *stream);

/* 64-bit FNV-1a over a byte string, continued from `h` (start with
 * APUS_FNV1A_INIT): the digest the token streams are compared by. */
#define APUS_FNV1A_INIT 0xcbf29ce484222325ull
uint64_t apus_fnv1a(const void *data, uint64_t nbytes, uint64_t h);

#ifdef __cplusplus
}
#endif
#endif /* APUS_SYNTH_H */
