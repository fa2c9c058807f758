// Test infrastructure (context rows only): a second entry point for the reference's im2col executable.
//
// The reference's own main (src_template/Ampere_FP16/im2col.cu:161-199) prints its average time as
// microseconds / 1e9 with "%f", i.e. always 0.000000, so the time of the im2col step cannot be read from its
// output.  This file compiles the unmodified reference source from where it lies (its path arrives as the macro
// REF_IM2COL), renames its main out of the way, and calls the same timing routine
// (testF16F16GemmPerformance, im2col.cu:108-159: `repeat` warm-up and `repeat` timed launches between CUDA events)
// with the same arguments, printing the microseconds per launch it returns.
#define main helix_reference_im2col_main
#include REF_IM2COL
#undef main

#include <cstdio>
#include <cstdlib>

int main(int argc, char** argv) {
  if (argc != 10) {
    std::fprintf(stderr, "usage: %s batch IC H W OC kH kW stride pad\n", argv[0]);
    return 2;
  }
  int v[9];
  for (int i = 0; i < 9; ++i) v[i] = std::atoi(argv[i + 1]);
  // argument order of the reference's call (im2col.cu:184-185): batch, IC, H, W, KH, OC, pad, stride, repeat
  const float us = testF16F16GemmPerformance(myF16F16GemmTCWarp<HGEMMAlignedV2>, v[0], v[1], v[2], v[3], v[5], v[4],
                                             v[8], v[7], 10);
  std::printf("%.3f\n", us);
  return 0;
}
