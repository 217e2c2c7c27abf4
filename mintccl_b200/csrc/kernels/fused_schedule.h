// Tile order of the tcgen05 GEMM kernels, plain and fused with a collective.  Host/device-agnostic so that the
// kernels (gemm_tc.cu: 128-row tiles, gemm_tc2.cu: 256-row tiles of a CTA pair) and the host model of the fused
// protocols (sim/sim_fused.cpp) walk exactly the same sequence.
//
//   plain              groups of `raster` row blocks, row block fastest inside a group: the tiles in flight at
//                      any time (consecutive t) span about as many rows of A as of B, which keeps the operands
//                      of a wave, and of the next one, inside the L2 for large problems (raster <= 1: row-major)
//   all-gather->GEMM   column blocks fastest; row blocks of rank r, r - 1, r - 2, ...: the order in which the
//                      peers' pushes arrive (every rank pushes to r + 1 first)
//   GEMM->reduce-scat. block j of every owner in turn, each rank starting at a different owner: the links stay
//                      balanced and block j of every owner is complete everywhere after (j + 1) / per of the
//                      run, so the reducers work alongside the GEMM instead of after it
//
// The reference has no compute kernels (README.md:5 only asks that collectives fuse with others).
#pragma once
#include "../device/sched.h"

#define MT_TILE_PLAIN 0
#define MT_TILE_AG_GEMM 1
#define MT_TILE_GEMM_RS 2

struct MtTile {
  int mb;     // row block of the tile in the whole problem (units of tile_rows)
  int nb;     // column block
  int owner;  // fused modes: rank that owns the rows (0 otherwise)
  int jb;     // fused modes: row block inside the owner's rows
};

MT_HD MtTile mt_fused_tile(int mode, int t, int M, int N, int nranks, int rank, int raster, int tile_rows, int tile_cols) {
  const int nbs = N / tile_cols;
  MtTile c;
  if (mode == MT_TILE_PLAIN) {
    const int mbs = M / tile_rows;
    const int G = raster > 1 ? raster : 1;
    const int per_group = G * nbs;
    const int g0 = (t / per_group) * G;
    const int gsz = (mbs - g0) < G ? (mbs - g0) : G;
    const int r = t % per_group;
    c.mb = g0 + r % gsz;
    c.nb = r / gsz;
    c.owner = 0;
    c.jb = c.mb;
    return c;
  }
  c.nb = t % nbs;
  const int mi = t / nbs;
  const int per = (M / nranks) / tile_rows;  // row blocks per rank
  int d;
  if (mode == MT_TILE_AG_GEMM) {
    d = mi / per;
    c.jb = mi % per;
    c.owner = mt_mod(rank - d, nranks);
  } else {
    c.jb = mi / nranks;
    d = mi % nranks;
    c.owner = mt_mod(rank + 1 + d, nranks);
  }
  c.mb = c.owner * per + c.jb;
  return c;
}
