// B200 launch table: (primitive, element bytes, input size) -> (threads, items, CTAs per SM).
// GENERATED from launch_table.json by tuning/gen_launch_table.py; edit the JSON, not this file.
// Rows of one (primitive, elem_bytes) group are ordered by ascending size bound and the first row
// whose bound covers the input wins; elem_bytes 0 matches any element size and closes a primitive.
#pragma once
#include <stdint.h>

namespace kf {
struct LaunchRow {
    int primitive;       // kf_primitive
    int elem_bytes;      // key+payload bytes for sorts; 0 = any
    uint64_t max_bytes;  // row applies to inputs of at most this many bytes
    int threads, items, blocks_per_sm;
};
static const LaunchRow kLaunchTable[] = {
    {0, 0, 18446744073709551615ull, 256, 4, 8},
    {1, 0, 16777216ull, 512, 4, 0},
    {1, 0, 18446744073709551615ull, 768, 4, 0},
    {2, 0, 18446744073709551615ull, 512, 16, 0},
    {3, 0, 18446744073709551615ull, 512, 16, 0},
};
static const int kNumLaunchRows = 5;
}  // namespace kf
