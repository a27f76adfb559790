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
