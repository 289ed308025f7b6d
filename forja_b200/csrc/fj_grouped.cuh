// Types shared by the expert-bucketed projection kernels (fj_grouped.cu, fj_grouped_tc5.cu).
#pragma once

#include "fj_kernels.h"

namespace fj {

// Up to tile_rows consecutive entries of the sorted route list, all of one expert.
struct RouteTile {
  unsigned expert, first, count;
};

struct GroupedArgs {
  const unsigned short* x;          // A source rows, bf16 [*, k]
  const unsigned* packed[2];        // [experts][n][k / 8]
  const unsigned short* scales[2];  // [experts][n][k / 64] bf16
  const unsigned short* biases[2];
  const unsigned* sorted;           // route ids bucketed by expert
  const RouteTile* tiles;
  const unsigned* n_tiles;
  void* out;                        // pair: bf16 [routes][n]; single: f32 (or bf16 when out_bf16) [routes][n]
  unsigned k, n, src_div;           // A row of a route = route / src_div
  int out_bf16;
};

// Tile GEMMs of 128 rows on the tcgen05 tensor cores (fj_grouped_tc5.cu); `tiles` = grid rows to launch.
bool grouped_tc5_supported(const GroupedArgs& a);
void launch_grouped_tc5(Ctx& ctx, const GroupedArgs& a, bool pair, unsigned tiles);
unsigned grouped_tc5_giveups();

}  // namespace fj
