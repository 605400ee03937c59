// Pieces shared by the grouped GEMM kernels: the ragged tile walker, the status recorder and
// small register-level helpers of the epilogues.
#pragma once
#include "../common/cam_types.h"
#include "../common/ptx.cuh"
#include "../common/quant.cuh"
#include "launch.h"

namespace cam {

constexpr int BM = 128, BN = 256, BK = 128, kStages = 4;
constexpr int kATile = BM * BK;            // 16 KiB
constexpr int kBTile = BN * BK;            // 32 KiB
constexpr int kStageBytes = kATile + kBTile;

// TM = rows of one tile along M (128 for one CTA per tile, 256 for a CTA pair).
template <int TM>
struct TileWalkerT {
    const int* off;
    int num_experts, n_tiles;
    int e, base;
    __device__ TileWalkerT(const int* o, int ne, int nt) : off(o), num_experts(ne), n_tiles(nt), e(0), base(0) {}
    // Maps a linear tile index (monotonically increasing across calls) to its expert and tile.
    // rot_den > 0: the row blocks of every expert are visited starting at block rot_num * blocks / rot_den (and wrapping
    // round).  The kernels whose epilogue pushes rows to the tokens' origin ranks pass (rank, ranks): an expert's rows are
    // ordered by origin rank, so without this every rank of the group would push to the same origin at the same time and
    // share that one GPU's ingress, one eighth of the link each on 8 GPUs.
    __device__ bool locate(int tile, int& e_out, int& mt, int& nt, int& row0, int& rows, int rot_num = 0, int rot_den = 0) {
        while (e < num_experts) {
            const int first = __ldg(off + e);
            const int cnt = __ldg(off + e + 1) - first;
            const int tiles = ((cnt + TM - 1) / TM) * n_tiles;
            if (tile < base + tiles) {
                const int local = tile - base;
                mt = local / n_tiles;
                nt = local - mt * n_tiles;
                if (rot_den > 0) {
                    const int blocks = (cnt + TM - 1) / TM;
                    mt += rot_num * blocks / rot_den;
                    if (mt >= blocks) mt -= blocks;
                }
                row0 = first + mt * TM;
                rows = min(TM, cnt - mt * TM);
                e_out = e;
                return true;
            }
            base += tiles;
            ++e;
        }
        return false;
    }
};

using TileWalker = TileWalkerT<BM>;

// A power-of-two scale as the word tcgen05 block scaling reads: its biased exponent (UE8M0 code) in all four bytes.
__device__ __forceinline__ uint32_t ue8m0_word(float scale) {
    return ((__float_as_uint(scale) >> 23) & 0xFFu) * 0x01010101u;
}
// The biased exponents (UE8M0 codes) of four power-of-two scales, one byte each: what the scale-factor warps of the
// block-scaled kernels make of a 16-byte load of four K-blocks' scales.  Byte i, replicated by __byte_perm(w, 0, 0x1111 * i),
// is the scale word of K-block i.
__device__ __forceinline__ uint32_t ue8m0_pack4(float a, float b, float c, float d) {
    return ((__float_as_uint(a) >> 23) & 0xFFu) | (((__float_as_uint(b) >> 23) & 0xFFu) << 8) |
           (((__float_as_uint(c) >> 23) & 0xFFu) << 16) | (((__float_as_uint(d) >> 23) & 0xFFu) << 24);
}
__device__ __forceinline__ uint32_t ue8m0_pack4(const float4& v) { return ue8m0_pack4(v.x, v.y, v.z, v.w); }

__device__ __forceinline__ void gemm_record_status(CamStatus* st, int code, int who, int detail) {
    if (atomicCAS(&st->code, 0, code) == 0) {
        st->who = who;
        st->detail = detail;
        st->block = static_cast<int>(blockIdx.x);
    }
}

// tcgen05.wait::ld that also names the destination registers, so no use of them can be
// scheduled ahead of the wait.
__device__ __forceinline__ void tc_wait_ld_regs(uint32_t (&v)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]),
                   "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]),
                   "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]),
                   "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]), "+r"(v[25]),
                   "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
                 :
                 : "memory");
}

__device__ __forceinline__ uint4 pack_bf16x8(float a0, float a1, float a2, float a3, float a4, float a5,
                                             float a6, float a7) {
    uint4 r;
    __nv_bfloat162 t0 = __floats2bfloat162_rn(a0, a1);
    __nv_bfloat162 t1 = __floats2bfloat162_rn(a2, a3);
    __nv_bfloat162 t2 = __floats2bfloat162_rn(a4, a5);
    __nv_bfloat162 t3 = __floats2bfloat162_rn(a6, a7);
    r.x = *reinterpret_cast<uint32_t*>(&t0);
    r.y = *reinterpret_cast<uint32_t*>(&t1);
    r.z = *reinterpret_cast<uint32_t*>(&t2);
    r.w = *reinterpret_cast<uint32_t*>(&t3);
    return r;
}

}  // namespace cam
