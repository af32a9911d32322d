// Host-side runtime shared by the C-ABI translation units: backend context,
// growable device workspaces, the weight cache keyed by host address, and the
// device-resident quantised-matrix handles.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "apus_b200.h"
#include "common.cuh"
#include "kernels.cuh"

namespace apus {

// A device buffer that only grows.  get() may reallocate (and then
// synchronises the device), so steady-state calls never allocate.
struct DevBuf {
    void *p = nullptr;
    size_t cap = 0;
    int get(size_t bytes, void **out);
    void release();
    template <class T> T *as() const { return static_cast<T *>(p); }
};

// One quantised matrix resident in HBM in the fragment-tiled layout.
struct DevQW {
    int fmt = 0;              // 4 or 8
    int O = 0, K = 0;
    uint8_t *codes = nullptr; // tiled codes
    uint8_t *scales = nullptr;// MXFP4: tiled scales; FP8: [O/128, K/128] bytes
    int zero_scale = 0;       // MXFP4 only
    bool owned = true;        // false when the storage belongs to a slab
    // FP8 on the tcgen05 kernel: codes stay in the reference storage [O, K]
    // (`codes` then points at it; owned == false when a device buffer of the
    // caller is used in place) and are read through this TMA tensor map
    bool tc = false;
    alignas(64) unsigned char map[128];
    std::map<int, GemmGroup *> tables;   // device work-item tables keyed by M
    size_t bytes() const;
    int table_for(int M, bool pair, const DevQW *other, GemmGroup **out, int *n_groups);
    void release();
};
}  // namespace apus

// The opaque handles of the C ABI are these runtime objects.
struct ApusCudaFp4 : apus::DevQW {};
struct ApusCudaFp8 : apus::DevQW {};

namespace apus {

struct Ctx {
    bool enabled = false;
    int device = 0;
    cudaStream_t stream = nullptr;          // the stream every entry point without a stream argument uses
    cudaStream_t own_stream = nullptr;      // the one the library created (stream may be the caller's)
    // side streams for independent kernel chains inside a step (joined back before
    // the step goes on); each has an event for the fork and one for the join
    static const int N_AUX = 5;
    cudaStream_t aux[N_AUX] = {};
    cudaEvent_t ev_fork[N_AUX] = {}, ev_join[N_AUX] = {};
    uint64_t bytes_uploaded = 0;
    std::unordered_map<const void *, DevQW *> qcache;      // quantised weights by host codes ptr
    std::unordered_map<const void *, DevBuf *> dcache;     // dense weights by host ptr
    std::unordered_map<const void *, ApusCudaMoe *> moes;  // MoE sublayers by host gate_w ptr
    DevBuf ws[16];                                         // host-tier workspaces
    DevBuf stage;                                          // upload staging
};
Ctx &ctx();
int ensure_enabled();
// aux stream i starts after everything enqueued on `main` so far / `main` waits for
// aux stream i.  Plain event dependencies, so they also work while `main` is
// being captured into a graph (the side chain becomes a parallel branch).
cudaStream_t branch_begin(cudaStream_t main, int i);
int branch_end(int i, cudaStream_t main);
// Files that keep device buffers outside Ctx register a release function
// (run by apus_cuda_disable) and optionally a per-host-pointer one (run by
// apus_cuda_forget).
void on_disable(void (*release_all)(), void (*forget_one)(const void *));

// Upload + re-tile one quantised matrix (host pointers in `codes`/`scales`).
int upload_qw(int fmt, const uint8_t *codes, const uint8_t *scales, int O, int K,
              uint8_t *dst_codes, uint8_t *dst_scales, int *zero_scale);
DevQW *new_qw(int fmt, const uint8_t *codes, const uint8_t *scales, int O, int K);
DevQW *cached_qw(int fmt, const uint8_t *codes, const uint8_t *scales, int O, int K);
const void *cached_dense(const void *host, size_t bytes);
bool is_device_ptr(const void *p);

// Quantised linear on device rows: act quant + block-scaled GEMM (+ BF16 round).
// `xq`/`xs` are caller workspaces of M*K bytes and M*K/128 floats.
int qlinear_dev(DevQW *w, const float *x, float *out, int M, uint8_t *xq, float *xs,
                bool round_out, cudaStream_t st);
// Block-scaled GEMM of pre-quantised rows against one matrix, or a gate/up pair
// with SwiGLU (`other` != NULL).
int qgemm_dev(DevQW *w, DevQW *other, const uint8_t *acodes, const float *ascales, int M, float *out,
              bool round_out, float limit, cudaStream_t st);
// SwiGLU expert on device rows (MXFP4 or FP8 by the handles' fmt).
struct ExpertWs { float *h; uint8_t *xq, *hq; float *xs, *hs; };
int expert_dev(DevQW *w1, DevQW *w2, DevQW *w3, float limit, const float *x, int rows,
               float *out, const ExpertWs &ws, cudaStream_t st);

}  // namespace apus
