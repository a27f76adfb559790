"""Transport rules of the comm layer (the device primitives are in csrc/comm.cuh).

Payload classes and their transport (mega_dsa_cp/comm/primitives.py:3-13 of the
reference):

* candidate lists, LSE scalars: 16-byte stores straight into every peer's arena;
* attention partials, compressor statistics: staged in shared memory, then one
  1-D bulk copy shared -> peer global per destination (`push_start`), completed
  later (`push_finish` = wait for the bulk group, then `fence.proxy.async`) so
  other work overlaps the transfer;
* flags: the event system; a notify follows the payload with release semantics
  at system scope, the consumer waits on the flag only and reads the payload
  with system-scope loads.
"""

PUSH_ALIGN = 16   # bulk copies want 16-byte aligned addresses and sizes


class DevicePrimitive:
    """A primitive that exists on the device only.  In the reference these names are CuTe-DSL functions
    called from inside CuTe kernels; here the kernels are CUDA C++ and the same primitives are the
    `cuda_symbol` of `header`.  The object documents the mapping and refuses a host-side call."""

    def __init__(self, name: str, cuda_symbol: str, header: str, ptx: str):
        self.__name__, self.cuda_symbol, self.header, self.ptx = name, cuda_symbol, header, ptx

    def __call__(self, *a, **k):
        raise RuntimeError(f"{self.__name__} is a device-side primitive: CUDA C++ kernels call {self.cuda_symbol} "
                           f"({self.header}); it cannot be called from the host")

    def __repr__(self):
        return f"<device primitive {self.__name__}: {self.cuda_symbol} in {self.header} -- {self.ptx}>"


_H, _C = "mega_dsa_cp_b200/csrc/comm.cuh", "mega_dsa_cp_b200/csrc/common.cuh"
cp_async_bulk_s2g = DevicePrimitive("cp_async_bulk_s2g", "mdc::bulk_s2g", _C, "cp.async.bulk.global.shared::cta.bulk_group")
cp_async_bulk_commit = DevicePrimitive("cp_async_bulk_commit", "mdc::bulk_commit", _C, "cp.async.bulk.commit_group")
cp_async_bulk_wait0 = DevicePrimitive("cp_async_bulk_wait0", "mdc::bulk_wait_all", _C, "cp.async.bulk.wait_group 0")
push_start = DevicePrimitive("push_start", "mdc::push_start", _H, "bulk copy shared -> (peer) global + commit_group")
push_finish = DevicePrimitive("push_finish", "mdc::push_finish", _H, "wait_group 0 + fence.proxy.async.global")
# NVLS multimem forms (re-exports of cutlass.utils.distributed in the reference): not used by these kernels,
# whose cross-rank payload travels by unicast P2P stores and bulk copies; the arena still carries the
# multicast address (mdc_peer_buffer.mc_base) for a caller's own kernels
multimem_st = DevicePrimitive("multimem_st", "(none: unicast stores, mdc::copy_to_peer)", _H, "multimem.st")
multimem_ld_reduce = DevicePrimitive("multimem_ld_reduce", "(none)", _H, "multimem.ld_reduce")
multimem_red_release_sys_add1 = DevicePrimitive("multimem_red_release_sys_add1", "(none: mdc::EventSet::notify_1t per peer)",
                                                "mega_dsa_cp_b200/csrc/events.cuh", "multimem.red.release.sys")
