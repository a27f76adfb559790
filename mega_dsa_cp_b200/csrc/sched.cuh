// Device side of the static task-DAG scheduler: every block stages its own
// queue row (int32 words, format of schedule/codegen.py) into shared memory
// once and walks it; a task entry carries its wait and notify edges inline.
//
//   entry  = [header][c0][c1][c2][wait event id]*[notify word]*
//   header = op | n_waits << 8 | n_notifies << 14 | extent_src << 20
//   notify = event id << 8 | destination rank ;  op 0xFF ends the row
//
// Wait target of an event = arity[event] * (phase + 1), phase = scalars[0],
// read once per launch: a launch can be replayed with only that scalar bumped.
// Device counterpart of mega_dsa_cp/schedule/device.py:35-129 of the reference.
#pragma once

#include "common.cuh"
#include "events.cuh"

namespace mdc {

constexpr int kOpEnd = 0xFF;

struct TaskInfo {
  int op, n_waits, n_notifies, extent_src;
  int c0, c1, c2;
  int pos;  // word offset of the header in the staged row
  __device__ bool valid() const { return op != kOpEnd; }
};

struct Cursor {
  const int32_t* row;  // staged queue row (shared memory)
  const unsigned long long* scalars;
  const int32_t* arity;
  const int32_t* scopes;
  unsigned long long phase;

  __device__ TaskInfo read(int pos) const {
    const int w = row[pos];
    TaskInfo t;
    t.op = w & 0xFF;
    t.n_waits = (w >> 8) & 0x3F;
    t.n_notifies = (w >> 14) & 0x3F;
    t.extent_src = (w >> 20) & 0xFF;
    t.c0 = row[pos + 1];
    t.c1 = row[pos + 2];
    t.c2 = row[pos + 3];
    t.pos = pos;
    return t;
  }
  __device__ TaskInfo advance(const TaskInfo& t) const { return read(t.pos + 4 + t.n_waits + t.n_notifies); }
  // dynamic trip-count bound of the task (0 when it has none)
  __device__ int extent(const TaskInfo& t) const {
    return t.extent_src ? static_cast<int>(scalars[t.extent_src] & 0xffffffffull) : 0;
  }
  __device__ int wait_event(const TaskInfo& t, int i) const { return row[t.pos + 4 + i]; }
  __device__ int notify_word(const TaskInfo& t, int i) const { return row[t.pos + 4 + t.n_waits + i]; }
  __device__ unsigned long long target(int ev) const {
    return static_cast<unsigned long long>(arity[ev]) * (phase + 1ull);
  }
};

}  // namespace mdc
