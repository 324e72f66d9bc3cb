// Exact (CUDA-core, float32 arithmetic) chunked SSD shared by the Mamba-2 and Mamba-3 entry points.
// One parameter block describes all three reference variants:
//   Mamba-2            m = 1, da = dt * A_h, source-column scale = dt, non-strict mask, D skip
//   Mamba-3 single     da given, source-column scale = scale, strict mask + gamma same-step term
//   Mamba-3 double     da given, no column scale, non-strict mask
#pragma once
#include "common.cuh"

namespace bm {
namespace exact {

struct Params {
    int B, S, H, P, R, G, M, Q, NC;
    int dtype;
    int strict;          // 1: same-time block weight = gamma (0 if gamma == NULL); 0: = column scale
    int cs_mode;         // 0: ones, 1: effective dt (Mamba-2), 2: `colscale` array
    int rope_dim, pairwise;
    const void* v;       // [b, s, m, h, p]
    const void* bmat;    // [b, s, m, G, r]
    const void* cmat;    // [b, s, m, G, r]
    const float* dsrc;   // [b, s, h]: dt (Mamba-2) or da (Mamba-3)
    const float* a;      // [h] or NULL: da = dsrc * a[h]
    const float* dt_bias;
    float dt_min, dt_max;
    const float* colscale;  // [b, s, h] (cs_mode 2)
    const float* gamma;     // [b, s, h] or NULL
    const float* d;         // [h] or NULL
    const float* h0;        // [b, h, p, r] or NULL
    const float* angles;    // [b, s, h, rope_dim/2] or NULL
    const void* z;          // [b, s, m, h, p] or NULL
    float* cum;             // workspace [b, h, nc, Q]
    float* cs;              // workspace [b, h, nc, Q]
    float* states;          // workspace or caller buffer [b, nc, h, p, r]
    void* y;
    float* h_final;
    float* gs;              // optional workspace [b, h, nc, Q]: same-time weight (written by K1 when set)
    int state_weight_mode;  // K3 row weight: 0 = cs * exp(Aend - cum) (forward), 1 = exp(cum) (readout gradient)
};

// Backward of the same general chunked SSD (Mamba-2 and both Mamba-3 cores).  All gradients float32.
struct BwdParams {
    Params fwd;             // forward inputs (y, h_final, z, angles, dt_bias unused / must be NULL)
    const void* dy;         // [b, s, m, h, p] act dtype
    const float* dh_final;  // [b, h, p, r] or NULL
    float* dv;              // [b, s, m, h, p]
    float* db;              // [b, s, m, G, r] (summed over the heads of a group when G < H)
    float* dc;              // [b, s, m, G, r]
    float* d_da;            // [b, s, h]   gradient of the per-step log-decay (Mamba-3: output; Mamba-2: internal)
    float* d_cs;            // [b, s, h]   gradient of the source-column scale (Mamba-3 single: d_scale)
    float* d_gs;            // [b, s, h]   gradient of the same-time weight   (Mamba-3 single: d_gamma)
    float* d_dt;            // [b, s, h]   Mamba-2 only: d_da * A + d_cs + d_gs
    float* d_a;             // [h]         Mamba-2 only: sum d_da * dt
    float* dd;              // [h] or NULL
    float* dh0;             // [b, h, p, r]
};

size_t bwd_workspace_bytes(int B, int S, int H, int P, int R, int Q, bool mamba2);
int32_t run_bwd(BwdParams p, void* workspace, size_t workspace_bytes, cudaStream_t stream);

size_t workspace_bytes(int B, int S, int H, int P, int R, int Q, bool need_states);
// Carves cum / cs / states out of `workspace` (states only if p.states == NULL on entry) and runs
// K1 -> K3 -> K4 -> K5 on `stream`.
int32_t run(Params p, void* workspace, size_t workspace_bytes, cudaStream_t stream);
// Same chain with the library's built-in scratch array instead of a caller workspace (no allocation).
int32_t run_noalloc(Params p, cudaStream_t stream);

}  // namespace exact
}  // namespace bm
