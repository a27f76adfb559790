// Latency probes of the event layer (CUDA counterparts of the reference's tests/bench_notify_latency.py:49-143):
// a ping-pong over two event cells, timed with %globaltimer on the pinging side, and the cost of a wait
// whose event is already complete.  Every wait is bounded; a wait that runs out is reported through the
// status block and ends the kernel.
#include "events.cuh"

namespace mdc {

// role 0: ping (notify `ev_ping` at `peer`, wait for own `ev_pong`), records one round-trip time per round;
// role 1: pong (wait for own `ev_ping`, notify `ev_pong` at `peer`);
// role 2: both roles in one launch on one GPU: block 0 pings, block 1 pongs (peer = own rank).
__global__ void __launch_bounds__(32) pingpong_kernel(const __grid_constant__ mdc_pingpong_params p) {
  if (threadIdx.x != 0) return;
  const EventSet ev{static_cast<unsigned char*>(p.events.base), p.events.offsets, p.events.my_rank, p.events.world};
  const int role = p.role == 2 ? static_cast<int>(blockIdx.x) : p.role;
  const bool sys = p.peer != ev.my_rank;
  for (int i = 0; i < p.rounds; ++i) {
    const unsigned long long want = p.base + static_cast<unsigned long long>(i) + 1ull;
    unsigned long long seen = 0;
    if (role == 0) {
      const unsigned long long t0 = global_timer_ns();
      ev.notify_1t(p.ev_ping, p.peer);
      if (!ev.poll_1t(p.ev_pong, want, sys, p.wait_budget_ns, &seen)) {
        report_failure(p.status, MDC_DEV_WAIT_TIMEOUT, p.ev_pong, i, seen, want);
        return;
      }
      if (p.out_ns) p.out_ns[i] = global_timer_ns() - t0;
    } else {
      if (!ev.poll_1t(p.ev_ping, want, sys, p.wait_budget_ns, &seen)) {
        report_failure(p.status, MDC_DEV_WAIT_TIMEOUT, p.ev_ping, i, seen, want);
        return;
      }
      ev.notify_1t(p.ev_pong, p.peer);
    }
  }
  if (role == 0 && p.out_ns) {  // cost of a wait on an event that is already complete (no hop involved)
    unsigned long long seen = 0;
    const unsigned long long t0 = global_timer_ns();
    for (int i = 0; i < 64; ++i) (void)ev.poll_1t(p.ev_pong, p.base + 1ull, sys, p.wait_budget_ns, &seen);
    p.out_ns[p.rounds] = (global_timer_ns() - t0) / 64;
  }
}

}  // namespace mdc

extern "C" int mdc_test_pingpong_launch(const mdc_pingpong_params* p, void* stream) {
  using namespace mdc;
  if (!p || !p->events.base || !p->events.offsets) return MDC_ERR_NULL;
  if (p->role < 0 || p->role > 2 || p->rounds < 1 || p->wait_budget_ns <= 0) return MDC_ERR_BAD_SHAPE;
  if (p->peer < 0 || p->peer >= p->events.world || p->ev_ping < 0 || p->ev_pong < 0 || p->ev_ping == p->ev_pong)
    return MDC_ERR_BAD_SHAPE;
  if (p->role == 2 && p->peer != p->events.my_rank) return MDC_ERR_BAD_SHAPE;
  pingpong_kernel<<<p->role == 2 ? 2 : 1, 32, 0, static_cast<cudaStream_t>(stream)>>>(*p);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}
