// Host-side declarations of the persistent decode kernel (decode_sm100.cu): embedding and every layer of
// one decode step of one sequence in ONE cooperative launch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace terb {

// Per-layer constants, an array in device memory (written when the model's weights are complete).
struct DecodeLayerDev {
    const uint8_t* W[7];      // internal strip layout, order q k v o gate up down
    float ws[7];              // per-tensor weight scales
    int pad_;
    const float* gamma[4];    // attn_norm, ffn_norm, attn_sub_norm, ffn_sub_norm (null: none)
    uint16_t* kcache;         // this layer's [B][Nkv][Smax][Hd] bf16
    uint16_t* vcache;
};

// Activations travel between the CTAs as flag-in-data words (tagged.cuh): one uint4 per pair of floats.
struct DecodeParams {
    const DecodeLayerDev* layers;
    const uint16_t* embd;     // bf16 [V][H]
    const int* tokens;        // [1]
    const int* pos;           // [1]
    float* hidden;            // [H] plain: the residual stream after the last layer (for the lm_head)
    uint4 *hid_t, *q_t, *k_t, *v_t, *att_t, *gate_t;   // tagged vectors: H/2, Hq/2, Hkv/2, Hkv/2, Hq/2, F/2 words
    uint4* rec_t;             // tagged attention partial records [Nh][max_chunks][Hd/2 + 1]
    unsigned* ctl;            // [0] step number (advanced by the step's last kernel), [1] abort mark
    const float* rope;        // [Smax][Hd/2][2]
    int* status;
    int L, H, F, Nh, Nkv, Hd, Smax, V, bitnet;
    float eps;
    unsigned long long wait_ns;   // limit of one wait on another CTA
    int poll_sleep_ns;        // pause between two looks at a value that has not arrived yet
    int fault_cta;            // test hook, -1 in normal use: this CTA does not publish its q/k/v of layer 0,
                              // so its consumers' waits run out (exercises the bounded-wait path)
    // set by the launcher
    int stages;               // ring depth per warp
    int x_bytes;              // bytes of the staged int8 activation vector (max Kpad)
    int tab_bytes;            // per-layer constants staged in shared memory
    int own_bytes;            // this CTA's columns of the residual stream (fp32) in shared memory
#ifdef TERB_TRACE
    unsigned long long* trace;    // diagnostic build only: [grid][32] timestamps of layer 1
#endif
};

// Words of the tagged state (hid, q, k, v, att, gate, records) and their offsets, in uint4 units.
struct DecodeStateLayout {
    size_t hid, q, k, v, att, gate, rec, total;
};
DecodeStateLayout decode_state_layout(int H, int F, int Nh, int Nkv, int Hd, int Smax);

// True when the persistent kernel covers this architecture (vector lengths that fit the register-resident
// quantiser, head dims 64/128, GQA groups 1/2/4/8).
bool decode_layers_supported(int H, int F, int Nh, int Nkv, int Hd, int L);
// Launches the kernel (cooperative: all CTAs are resident; they hand values to each other while running).
cudaError_t launch_decode_layers(const DecodeParams& p, int sm_count, cudaStream_t st);

}  // namespace terb
