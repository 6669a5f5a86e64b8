// Shared-memory tile geometry of the register-patch kernels (step_fast.cu, step_bwd_fast.cu).
//
// A CTA of 128 threads always owns an 8 x 8 x 8 region of the grid; thread (xp, yp, z) owns the
// 1 x 2 x 2 patch at (z, 2 yp, 2 xp) of the region. With block size 8 the region is one block and
// its tile is the 10 x 10 x 10 neighbourhood. With block size 4 the region holds eight blocks,
// each with its own 6 x 6 x 6 tile (the halo of a block is stale even where it overlaps a
// neighbouring block of the same region), laid out one after the other. The strides are chosen so
// that the 64-bit window loads of a half-warp touch every bank once:
//   block 8: rows of 12 floats, planes of 120;
//   block 4: rows of 8, planes of 54, sub-tiles of 324 (= 4 mod 32): the 16 lanes of a half-warp
//            differ in (xp & 1, xp >> 1, yp & 1, yp >> 1), which move the address by 2, 324, 16
//            and 648 floats, i.e. by 1, 2, 8 and 4 eight-byte bank pairs.
#pragma once

namespace gn {

template <int SUB>
struct PatchGeo;

template <>
struct PatchGeo<8> {
    static constexpr int RS = 12, PS = 120, TS = 1200;
    static constexpr int CELLS = 1000;     // tile cells fetched per sample
    static constexpr int SLOTS = 8;        // ceil(CELLS / 128)
    static constexpr int SOFF_BITS = 11;   // bits of a tile offset inside a cell descriptor
    __device__ static int window_origin(int xp, int yp, int z) { return z * PS + 2 * yp * RS + 2 * xp; }
    // cell i of the fetch list: tile offset, coordinates inside the region's 10^3 neighbourhood,
    // and whether it is a halo cell of its block
    __device__ static void cell(int i, int &soff, int &cz, int &cy, int &cx, bool &halo)
    {
        cx = i % 10, cy = (i / 10) % 10, cz = i / 100;
        soff = cz * PS + cy * RS + cx;
        halo = cx == 0 || cx == 9 || cy == 0 || cy == 9 || cz == 0 || cz == 9;
    }
};

template <>
struct PatchGeo<4> {
    static constexpr int RS = 8, PS = 54, SUB_TS = 324, TS = 8 * SUB_TS;
    static constexpr int CELLS = 8 * 216;
    static constexpr int SLOTS = 14;
    static constexpr int SOFF_BITS = 12;
    __device__ static int window_origin(int xp, int yp, int z)
    {
        const int sub = ((z >> 2) * 2 + (yp >> 1)) * 2 + (xp >> 1);
        return sub * SUB_TS + (z & 3) * PS + 2 * (yp & 1) * RS + 2 * (xp & 1);
    }
    __device__ static void cell(int i, int &soff, int &cz, int &cy, int &cx, bool &halo)
    {
        const int sub = i / 216, l = i % 216;
        const int lz = l / 36, ly = (l / 6) % 6, lx = l % 6;
        soff = sub * SUB_TS + lz * PS + ly * RS + lx;
        cz = (sub >> 2) * 4 + lz, cy = ((sub >> 1) & 1) * 4 + ly, cx = (sub & 1) * 4 + lx;
        halo = lx == 0 || lx == 5 || ly == 0 || ly == 5 || lz == 0 || lz == 5;
    }
};

}  // namespace gn
