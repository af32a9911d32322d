// Checkpoint directory reader (host side): config.json, the safetensors shard
// index and the shards' payloads, read with positional I/O.  No device code.
#pragma once
#include <stdint.h>
#include <atomic>
#include <map>
#include <string>
#include <vector>
#include "apus_b200.h"

namespace apus {

struct CkTensor {
    std::string name;
    int dtype = APUS_CUDA_ST_OTHER, ndim = 0;
    int64_t shape[8] = {0};
    int shard = -1;
    uint64_t off = 0, nbytes = 0;          // absolute file offset of the payload
    uint64_t nelem() const { uint64_t n = 1; for (int d = 0; d < ndim; d++) n *= (uint64_t)shape[d]; return n; }
};

struct CkShard {
    std::string file;
    int fd = -1;
    bool parsed = false;
    std::vector<CkTensor> tensors;
    std::map<std::string, int> by_name;
};

}  // namespace apus

struct ApusCudaCkpt {
    std::string dir, wdir;                  // wdir: where the index and the shards lie
    ApusCudaCkptCfg cfg;
    // the DSpark section of the config (c/model.h:48-56, 336-373); valid when cfg.dspark
    int ds_block = 0, ds_noise = 0, ds_rank = 0, ds_stages = 0, ds_ntargets = 0, ds_targets[8] = {0};
    std::vector<int> ratios, hash;
    std::vector<apus::CkShard> shards;
    std::map<std::string, int> shard_of;    // tensor name -> shard
    std::atomic<uint64_t> reads{0}, read_bytes{0};

    // NULL + message when the tensor is not in the index or its shard is unreadable
    const apus::CkTensor *find(const std::string &name, std::string *why);
    int read_at(int shard, uint64_t off, void *dst, uint64_t n, std::string *why);
    int read(const apus::CkTensor &t, void *dst, std::string *why) { return read_at(t.shard, t.off, dst, t.nbytes, why); }
    ~ApusCudaCkpt();
};

namespace apus {

// One layer's tensors in host memory, laid out as the reference's loader leaves
// them (c/layer.h:202-330), and the descriptor that points at them.
struct CkLayerHost {
    std::vector<std::vector<uint8_t>> raw;          // quantised payloads and expert slabs
    std::vector<std::vector<float>> f32;
    std::vector<uint16_t> wo_a;
    std::vector<int64_t> tid2eid;
    std::vector<ApusFp4W> w1, w2, w3;
    ApusCudaLayerDesc desc;
};
// Experts outside [e_lo, e_hi) are not read (their views stay NULL).
int ckpt_load_layer(ApusCudaCkpt *c, int layer, int e_lo, int e_hi, CkLayerHost *out, std::string *why);
int ckpt_load_layer_named(ApusCudaCkpt *c, const std::string &prefix, int ratio, int hash, int layer, int e_lo, int e_hi,
                          CkLayerHost *out, std::string *why);
int ckpt_rope(const ApusCudaCkptCfg &cfg, int ratio, int64_t rows, float *cos, float *sin);

}  // namespace apus
