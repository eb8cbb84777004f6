// Interface of the two-CTA (tcgen05.mma.cta_group::2) bf16 / f16 GEMM kernel, launched by matmul_tc.cu with tensor
// maps it has built: A boxes of BM rows (K-major) or 64 x 64 chunks (MN-major), B boxes of BN_HALF rows or 64 x 64
// chunks, D boxes of 32 rows x 64 columns (32 f32 columns for split-K partials).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace mx {
namespace tc2 {

constexpr int BM = 128;       // rows of A and of the output per CTA; a pair covers 256
constexpr int BN = 256;       // columns of the pair's tile
constexpr int BN_HALF = 128;  // columns of B each CTA stages
constexpr int BK = 64;

struct Params {
    int tile_pairs_m, tiles_n;   // row-tile pairs (256 rows each) and column tiles
    int tiles_per_batch;         // tile_pairs_m * tiles_n
    int num_tiles;               // batch * tiles_per_batch (pair tiles)
    int num_kb;
    int a_batched, b_batched;
    int is_bf16, out_f32;
    int a_mn, b_mn;
};

// `ctas`: CTAs the launch may use (rounded down to whole pairs).  Returns false when the kernel cannot be launched
// (then nothing was queued and the caller uses the one-CTA kernel).
bool launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_d, const Params& p, int ctas, int* err, int tag,
            cudaStream_t stream);

// Pairs of CTAs of the kernel that can be resident at once on the current device; -1 when the query fails.
int max_resident_pairs();

}  // namespace tc2
}  // namespace mx
