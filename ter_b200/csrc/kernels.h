// Host-side declarations of the kernel launchers (implemented in the .cu files).
// Every launcher returns a cudaError_t and launches on the given stream.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace terb {

// ---- internal weight layout -------------------------------------------------
// Bytes [Npad/4][Kpad]: byte-column jb holds columns 4*jb..4*jb+3 for consecutive k
// (the reference's v11 arrangement, cuda/ter_cuda_forward_packed.cu:354-355), with
//   * the 2-bit field re-coded to u = trit + 1 (0 -> -1, 1 -> 0, 2 -> +1), so that a
//     masked word is directly an unsigned dp4a operand,
//   * K padded to a multiple of 128 with u = 1 (trit 0), N padded to a multiple of 16.
// A "tile" is 4 consecutive byte-columns (16 output columns): 4*Kpad contiguous bytes.
struct DevWeight {
    uint8_t* data = nullptr;
    int K = 0, N = 0, Kpad = 0, Npad = 0;
    float scale = 0.f;
    size_t bytes() const { return (size_t)(Npad / 4) * (size_t)Kpad; }
    int tiles() const { return Npad / 16; }
};

constexpr int kGemvMaxGroup = 4;
constexpr int kGemvMaxK = 32768;

struct GemvParams {
    const uint8_t* W[kGemvMaxGroup];
    float* out[kGemvMaxGroup];
    int32_t* acc_out[kGemvMaxGroup];
    float w_scale[kGemvMaxGroup];
    int N[kGemvMaxGroup];
    int tile_begin[kGemvMaxGroup + 1];
    const int8_t* x;
    const float* x_scale;   // device scalar; when null, x_scale_imm is used
    float x_scale_imm;
    int K, Kpad;
    int n_mats, n_tiles, stages;
    int* status;
};

struct GemvLaunchCfg {
    int ctas_per_sm = 4;
    int stages = 0;      // 0 = choose from the tile size
    int pdl = 1;
    int sm_count = 148;
};

cudaError_t launch_gemv(const GemvParams& p, const GemvLaunchCfg& cfg, cudaStream_t st);

// ---- install-time re-pack (device side) --------------------------------------
cudaError_t launch_recode_v11(const uint8_t* src, uint8_t* dst, int K, int N, int Kpad, int Npad, cudaStream_t st);
cudaError_t launch_recode_rowmajor(const uint8_t* src, uint8_t* dst, int K, int N, int Kpad, int Npad, cudaStream_t st);
// bad_count receives the number of payload values outside {-1,0,+1}.
cudaError_t launch_pack_i32(const int32_t* src, uint8_t* dst, int K, int N, int Kpad, int Npad, int* bad_count,
                            cudaStream_t st);

}  // namespace terb
