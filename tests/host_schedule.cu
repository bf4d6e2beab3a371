// Host-side access to the tensor-core kernels' work-unit decoder (decode_unit_on, tc_device.cuh), for the CPU test
// of the schedules (tests/test_schedule.py): every unit of a launch is decoded exactly as a CTA would decode it.
#include "../dfdx_b200/csrc/tc_device.cuh"

using namespace b200::tcx;

// out: total_units rows of (tile, kb_lo, kb_hi).  The schedule is given by the same fields the launchers set.
extern "C" int schedule_units(long long total_tiles, int total_kb, long long grid, long long total_units, int ksplit,
                              int kb_per_slice, int streamk, long long sk_per_cta, long long tail_from, int tail_per,
                              int kt_cut, int kt_per, long long* out) {
  TcArgs g = {};
  g.total_tiles = total_tiles; g.total_units = total_units;
  g.ksplit = ksplit; g.kb_per_slice = kb_per_slice;
  g.streamk = streamk; g.sk_per_cta = sk_per_cta;
  g.tail_from = tail_from; g.tail_per = tail_per; g.tail_parts = 2;
  g.kt_cut = kt_cut; g.kt_per = kt_per;
  for (long long u = 0; u < total_units; ++u) {
    const Unit un = decode_unit_on(g, u, total_kb, grid);
    out[3 * u] = un.tile; out[3 * u + 1] = un.kb_lo; out[3 * u + 2] = un.kb_hi;
  }
  return 0;
}
