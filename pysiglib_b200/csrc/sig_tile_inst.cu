// One part of the register-tile kernel table (tile_table.h).  This file is compiled
// SIG_TILE_PARTS times with -DSIG_TILE_PART=<k> so the variants build in parallel.
#include "sig_tile_launch.cuh"
#ifndef SIG_TILE_TABLE
#define SIG_TILE_TABLE "tile_table.h"  // -DSIG_TILE_TABLE='"other.h"': a table restricted to the shapes a deployment needs
#endif
#include SIG_TILE_TABLE

#ifndef SIG_TILE_PART
#error "compile with -DSIG_TILE_PART=<k>"
#endif

#define SIG_CAT2(a, b) a##b
#define SIG_CAT(a, b) SIG_CAT2(a, b)

namespace sigb200 {

void SIG_CAT(register_tile_part_, SIG_TILE_PART)(std::vector<TileEntry>& table) {
#define X(T, BWD, D, N, P, G, EST, LOG) table.push_back(make_tile_entry<T, D, N, P, G, BWD, LOG>(EST));
    SIG_CAT(SIG_TILE_PART_, SIG_TILE_PART)(X)
#undef X
}

}  // namespace sigb200
