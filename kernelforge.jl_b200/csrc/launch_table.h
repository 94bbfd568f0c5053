// B200 launch table: (primitive, element bytes, input size) -> (threads, items, CTAs per SM).
// GENERATED from tuning/launch_table.json by tuning/gen_launch_table.py; edit the JSON, not this file.
// The first row that matches the primitive and element size and whose bound covers the input wins;
// elem_bytes 0 matches any element size (key + payload bytes for sorts).
#pragma once
#include <stdint.h>

namespace kf {
struct LaunchRow {
    int primitive;       // kf_primitive
    int elem_bytes;      // 0 = any
    uint64_t max_bytes;  // row applies to inputs of at most this many bytes
    int threads, items, blocks_per_sm;
};
static const LaunchRow kLaunchTable[] = {
    {0, 0, 1048576ull, 256, 4, 1},
    {0, 0, 16777216ull, 256, 4, 4},
    {0, 0, 18446744073709551615ull, 512, 4, 4},
    {1, 0, 4194304ull, 256, 8, 0},
    {1, 8, 18446744073709551615ull, 512, 8, 0},
    {1, 2, 18446744073709551615ull, 512, 8, 0},
    {1, 4, 18446744073709551615ull, 384, 8, 0},
    {1, 0, 18446744073709551615ull, 768, 4, 0},
    {2, 4, 18446744073709551615ull, 512, 24, 0},
    {2, 0, 18446744073709551615ull, 512, 16, 0},
    {3, 0, 18446744073709551615ull, 512, 16, 0},
};
static const int kNumLaunchRows = 11;
}  // namespace kf
