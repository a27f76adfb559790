"""CPU checks of the C-ABI library (it loads, exports every symbol the header
declares, rejects bad arguments without touching a GPU), of the import alias,
and of the multi-rank host logic (gloo, world size 2)."""

import ctypes as C
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "mdc.h")).read()
    return sorted(set(re.findall(r"^\s*(?:int|const char\*)\s+(mdc_\w+)\s*\(", text, flags=re.M)))


def test_library_exports_every_declared_symbol():
    from mega_dsa_cp_b200 import _native as N

    lib = N.lib()
    declared = _declared_symbols()
    assert len(declared) >= 16
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/mdc.h but not exported"
    assert sorted(N.EXPORTS) == declared
    assert lib.mdc_abi_version() == N.ABI_VERSION
    assert lib.mdc_status_string(-1).decode() != lib.mdc_status_string(-4).decode()


def test_launchers_reject_bad_arguments_without_a_gpu():
    from mega_dsa_cp_b200 import _native as N

    lib = N.lib()
    assert lib.mdc_logits_fp4_launch(None, None) == -4
    p = N.LogitsParams()
    assert lib.mdc_logits_fp4_launch(C.byref(p), None) == -4          # null pointers
    p.kv_pages = p.q = p.weights = p.block_table = p.logits = 4096
    p.fmt, p.q_fmt, p.page_tokens, p.heads, p.q_len = 7, 1, 64, 64, 1
    assert lib.mdc_logits_fp4_launch(C.byref(p), None) == -3          # unknown format
    p.fmt, p.page_tokens = N.FMT_MXFP4, 64
    assert lib.mdc_logits_fp4_launch(C.byref(p), None) == -1          # mxfp4 needs 128-token pages
    m = N.MergeTopkParams()
    assert lib.mdc_merge_topk_launch(C.byref(m), None) == -4
    l = N.LseMergeParams(acc_o=4096, acc_lse=4096, o=4096, rows=1, H=128, D=512, n_slices=17, n_slices_max=17)
    assert lib.mdc_lse_merge_launch(C.byref(l), None) == -1           # more slices than supported
    a = N.SparseMlaParams(q=4096, kv_cmp=4096, pt_cmp=4096, k_valid=4096, o=4096, B=1, q_len=1, H=100)
    assert lib.mdc_sparse_mla_launch(C.byref(a), None) == -1          # heads not a multiple of 64
    c = N.CompressParams()
    assert lib.mdc_compress_step_launch(C.byref(c), None) == -4
    assert lib.mdc_megakernel_launch(None, None) == -4
    assert lib.mdc_megakernel_threads() in (448, 576) and lib.mdc_megakernel_smem_bytes() > 200 * 1024


def _valid_mega_params(N, cp=1, attn_splits=1, bpc=128, heads=128, top_k=2048, layer=True):
    """Parameters mdc_megakernel_check accepts (fake 4096-aligned addresses: nothing is dereferenced)."""
    A = 1 << 20
    p = N.MegaParams()
    p.queue = p.scalars = p.arity = p.scopes = A
    p.row_words, p.n_ctas, p.n_events, p.wait_budget_ns = 8, 4, 1, 1000
    p.events = N.EventSetC(A, A, 0, cp)
    p.arena = N.PeerBufferC(A, A, 0, cp, 0)
    if not layer:
        return p
    B = 4
    lp = N.LogitsParams(kv_pages=A, num_pages=64, page_tokens=64, fmt=N.FMT_NVFP4, q_fmt=N.Q_BF16, q=A, weights=A,
                        block_table=A, max_pages=256, cand_v=A, cand_i=A, cand_c=A, top_k=top_k, B=B, q_len=1,
                        heads=64, blocks_per_chunk=bpc, n_chunks=2, id_mul=cp, id_add=0)
    mp = N.SparseMlaParams(q=A, kv_cmp=A, pt_cmp=A, k_valid=A, o=A, lse=A, o_stride=heads * 512, lse_stride=heads,
                           B=B, q_len=1, H=heads, d_qk=576, d_v=512, pages_cmp=1000, page_cmp=1, pt_cols=top_k,
                           kv_dtype=N.DT_BF16, out_dtype=N.DT_BF16, n_splits=1, softmax_scale=0.04, output_scale=1.0)
    L = N.LayerParams()
    L.cp, L.rank, L.B, L.top_k, L.H, L.n_chunks = cp, 0, B, top_k, heads, 2
    L.kv_seq_stride, L.attn_splits, L.logits, L.mla = 16384, attn_splits, lp, mp
    L.phase_bytes, L.phases = 1 << 20, 2
    L.sel_v = L.sel_i = L.sel_c = L.out = L.out_lse = A
    L.out_dtype, L.l1_groups = N.DT_BF16, 1
    p.layer = L
    return p


def test_megakernel_check_rejects_bad_layer_configurations():
    """Configurations that would overrun on-chip arrays or dereference missing buffers come back as
    error codes from the host-side check (no GPU involved)."""
    from mega_dsa_cp_b200 import _native as N

    chk = lambda p: N.lib().mdc_megakernel_check(C.byref(p))
    assert chk(_valid_mega_params(N)) == 0
    assert chk(_valid_mega_params(N, layer=False)) == 0               # test queues carry no layer
    assert chk(_valid_mega_params(N, cp=8, attn_splits=2)) == 0       # 16 LSE slices: the limit
    assert chk(_valid_mega_params(N, cp=8, attn_splits=4)) == -6      # 32 slices overrun the merge's arrays
    assert chk(_valid_mega_params(N, bpc=1024)) == -6                 # 65536 scores per chunk: past the kernel's shared memory
    assert chk(_valid_mega_params(N, heads=96)) == -1                 # heads not a multiple of 64
    assert chk(_valid_mega_params(N, top_k=2047)) in (-1, -2)         # candidate slice not a multiple of 16 bytes
    p = _valid_mega_params(N)
    p.layer.sel_i = None
    assert chk(p) == -4
    p = _valid_mega_params(N)
    p.layer.l1_groups = 2                                             # two-level merge without its scratch
    assert chk(p) == -4
    p = _valid_mega_params(N)
    p.layer.logits.kv_pages = None                                    # the indexer tile's own check
    assert chk(p) == -4
    p = _valid_mega_params(N)
    p.layer.mla.d_qk = 500                                            # the attention tile's own check
    assert chk(p) == -1
    p = _valid_mega_params(N)
    p.layer.rank = 3                                                  # rank outside cp
    assert chk(p) == -1
    p = _valid_mega_params(N)
    p.arena = N.PeerBufferC(None, None, 0, 1, 0)                      # a layer needs the arena
    assert chk(p) == -4
    # the exact row selection and the candidate exchange variants
    A = 1 << 20
    def exact(cp, mode, direct):
        p = _valid_mega_params(N, cp=cp)
        p.layer.thr_hist = p.layer.thr_done = A
        p.layer.thr_exact, p.layer.thr_ev_base, p.layer.thr_off, p.layer.cand_direct = mode, p.n_events, 4096, direct
        return p
    assert chk(exact(1, 1, 0)) == 0 and chk(exact(2, 1, 1)) == 0 and chk(exact(2, 2, 0)) == 0
    assert chk(exact(2, 1, 0)) == -1          # across ranks the selection is published through the chunk lists' layout
    assert chk(exact(2, 2, 1)) == -1          # ... and a rank's own exact list is one list per rank
    assert chk(exact(1, 3, 0)) == -1
    p = exact(1, 1, 0)
    p.layer.thr_hist = None                   # no row histogram
    assert chk(p) == -1
    p = exact(1, 1, 0)
    p.layer.thr_ev_base = 0                   # the extra event cells must lie behind the queue's events
    assert chk(p) == -1
    p = _valid_mega_params(N, cp=2, top_k=2046)
    p.layer.cand_direct = 1                   # the ids of a slice start on a 16-byte boundary
    assert chk(p) in (-1, -2)
    p = _valid_mega_params(N)
    p.layer.kv_group = -1
    assert chk(p) == -1
    p = _valid_mega_params(N)
    p.dyn_task_off, p.dyn_n_tasks = A, 4      # dynamic scheduling without its counters
    assert chk(p) == -4
    # and the Python layer object refuses the same things before it builds anything
    from mega_dsa_cp_b200.layer import DsaDecodeLayer
    with pytest.raises(AssertionError):
        DsaDecodeLayer(4, cp=8, rank=0, attn_splits=4, device="cpu", n_ctas=8)


def test_missing_library_fails_loudly(tmp_path):
    code = ("import os, sys; sys.path.insert(0, %r); os.environ['MDC_LIB_PATH'] = %r\n"
            "from mega_dsa_cp_b200 import _native\n"
            "try:\n    _native.lib()\nexcept _native.MdcError as e:\n    print('LOUD', 'no fallback' in str(e))\n"
            % (ROOT, str(tmp_path / "nope.so")))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert "LOUD True" in r.stdout, r.stdout + r.stderr


def test_reference_import_paths_resolve():
    import mega_dsa_cp.tiles.logits as a
    import mega_dsa_cp_b200.tiles.logits as b
    from mega_dsa_cp.comm.buffers import alloc_arena  # noqa: F401
    from mega_dsa_cp.events.symm import alloc_event_buffer  # noqa: F401
    from mega_dsa_cp.tiles.fp4 import make_index_cache, quant_mxfp4  # noqa: F401
    from mega_dsa_cp.tiles.hca import run_hca_fp8  # noqa: F401
    from mega_dsa_cp.tiles.lse_merge import run_lse_merge  # noqa: F401
    from mega_dsa_cp.tiles.merge import run_merge_topk  # noqa: F401

    assert a.run_fp4_paged_mqa_logits is b.run_fp4_paged_mqa_logits


def test_package_fp4_helpers_match_oracle():
    from mega_dsa_cp_b200.tiles import fp4
    from oracle import dsa_oracle as orc

    g = torch.Generator().manual_seed(0)
    x = torch.randn(256, 128, generator=g) * torch.logspace(-2, 1.5, 256).unsqueeze(1)
    for mine, theirs in ((fp4.quant_mxfp4, orc.quant_mxfp4), (fp4.quant_nvfp4, orc.quant_nvfp4)):
        a, b = mine(x), theirs(x)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    pk, sf = fp4.quant_mxfp4(x)
    assert torch.equal(fp4.dequant_mxfp4(pk, sf), orc.dequant_fp4(pk, sf, "mxfp4"))
    pk, sf = fp4.quant_nvfp4(x)
    assert torch.equal(fp4.dequant_nvfp4(pk, sf), orc.dequant_fp4(pk, sf, "nvfp4"))
    assert torch.equal(fp4.sf_to_atom(sf[:, :4].contiguous()), orc.sf_to_atom(sf[:, :4].contiguous()))
    for fmt, P in (("mxfp4", 128), ("nvfp4", 64), ("nvfp4", 128)):
        f1, _ = fp4.fuse_pages(x, fmt, P)
        f2, _ = orc.build_index_pages(x, fmt, P)
        assert torch.equal(f1, f2) and f1.shape[1] == fp4.page_bytes(fmt, P)
    kv, sfp = fp4.make_index_cache(2, 2, device="cpu", seed=0)
    assert kv.shape == (4, 8704) and sfp.shape == (4, 128, 4)
    qp, qsf, qatom, w = fp4.make_q(2, q_len=1, device="cpu")
    assert qp.shape == (2, 64, 64) and qatom.shape == (2, 512) and w.shape == (2, 64)


WORKER = r'''
import os, sys, json
sys.path.insert(0, %(root)r)
import torch, torch.distributed as dist
from mega_dsa_cp_b200.layer import build_layer_dag, arena_regions
from mega_dsa_cp_b200.schedule.codegen import codegen_schedule
from mega_dsa_cp_b200.comm.buffers import layout_regions
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
tasks, events, ops = build_layer_dag(B=6, n_chunks=3, cp=world, heads=128)
s = codegen_schedule(tasks, events, rank=rank, n_ctas=5, world_size=world, op_of=ops)
# every rank derives the same event tables; arities differ only by ownership
mine = torch.tensor(s.arity + s.scopes + [s.n_events], dtype=torch.int64)
gathered = [torch.zeros_like(mine) for _ in range(world)]
dist.all_gather(gathered, mine)
n = s.n_events
ok = all(torch.equal(g[n:], mine[n:]) for g in gathered)               # scopes and count identical
part = [4 * b + 3 for b in range(6)]
for r, g in enumerate(gathered):                                        # part[b] arity only on the owner
    ok &= all((int(g[e]) > 0) == (b %% world == r) for b, e in enumerate(part))
offs, per_phase = layout_regions(arena_regions(6, world, 2048))
ok &= offs["cand"] == 0 and offs["inbox"] %% 256 == 0 and per_phase %% 256 == 0
n_tasks = sum(1 for t in tasks if t.rank == rank)
ok &= len(s.topo) == n_tasks
flag = torch.tensor([1 if ok else 0]); dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0: print("HOST_OK" if flag.item() == 1 else "HOST_FAIL")
dist.destroy_process_group()
'''


def test_layer_dag_two_ranks_gloo(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(WORKER % {"root": ROOT})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29611", str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert "HOST_OK" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]


@pytest.mark.parametrize("n_chunks,cp,splits", [(2, 1, 1), (4, 2, 2), (8, 2, 4), (16, 4, 1), (5, 8, 2), (20, 1, 1)])
def test_layer_dag_variants_validate(n_chunks, cp, splits):
    """Two-level local merge (more than 8 chunks), attention slot splits and the four LSE head
    groups: every variant is a valid DAG on every rank, with the arities the kernels rely on."""
    from mega_dsa_cp_b200.events import validate
    from mega_dsa_cp_b200.layer import LSE_GROUPS, arena_regions, build_layer_dag, l1_groups_for
    from mega_dsa_cp_b200.schedule.codegen import codegen_schedule

    B, heads = 5, 128
    G = l1_groups_for(n_chunks)
    assert (G == 1) == (n_chunks <= 8) and (G == 1 or G * 4 >= n_chunks)
    tasks, events, ops = build_layer_dag(B, n_chunks, cp, heads, splits, G)
    errors, table = validate(tasks, events, cp)
    assert not errors, errors[:3]
    for r in range(cp):
        s = codegen_schedule(tasks, events, rank=r, n_ctas=7, world_size=cp, op_of=ops)
        mine = [t for t in tasks if t.rank == r]
        assert len(s.topo) == len(mine)
        names = {e.name: i for i, e in enumerate(events)}
        for b in range(B):
            # part[b] is notified by every rank's attention tasks, only into its owner
            want = cp * 4 * splits if b % cp == r else 0
            assert s.arity[names[f"part[{b}]"]] == want
            assert s.arity[names[f"l1[{b}]"]] == (G if G > 1 else n_chunks)
            if cp > 1:
                assert s.arity[names[f"cand[{b}]"]] == cp
            else:   # one rank: MERGE_L1 publishes the selection itself, no candidate exchange and no MERGE_L2
                assert f"cand[{b}]" not in names and not any(t.name.startswith("merge_l2") for t in mine)
        n_lse = sum(1 for t in mine if t.name.startswith("lse_merge"))
        assert n_lse == LSE_GROUPS * sum(1 for b in range(B) if b % cp == r)
    # the optional task families (query distribution, new-token write, compressor) keep the DAG valid
    tasks, events, ops = build_layer_dag(B, n_chunks, cp, heads, splits, 1, compressor=True, qpath=True, kvwrite=True)
    errors, _ = validate(tasks, events, cp)
    assert not errors, errors[:3]
    for r in range(cp):
        codegen_schedule(tasks, events, rank=r, n_ctas=7, world_size=cp, op_of=ops)
    # several ranks, chunk lists stored by the LOGITS tasks themselves: no MERGE_L1, cand[b] counts cp x chunks
    for qp in (False, True):
        tasks, events, ops = build_layer_dag(B, n_chunks, cp, heads, splits, 1, qpath=qp, cand_direct=True)
        errors, _ = validate(tasks, events, cp)
        assert not errors, errors[:3]
        names = {e.name: i for i, e in enumerate(events)}
        for r in range(cp):
            s = codegen_schedule(tasks, events, rank=r, n_ctas=7, world_size=cp, op_of=ops)
            has_l1 = any(t.name.startswith("merge_l1") for t in tasks if t.rank == r)
            assert has_l1 == (cp == 1)
            if cp > 1:
                assert all(s.arity[names[f"cand[{b}]"]] == cp * n_chunks for b in range(B))
                assert ("l1[0]" in names) == qp
    reg = arena_regions(B, cp, 2048, heads, splits)
    assert reg["inbox"] == -(-B // cp) * cp * splits * (heads * 512 * 2 + heads * 4)
    assert arena_regions(B, cp, 2048, heads, splits, cand_lists=n_chunks)["cand"] == n_chunks * reg["cand"]


def test_prefill_causal_lengths_and_dense_tables():
    """Host arithmetic of the chunked prefill (token t lives on rank t % cp at local index t // cp) and of the
    dense-layer page tables."""
    import torch

    from mega_dsa_cp_b200.prefill import causal_local_lens
    from mega_dsa_cp_b200.tiles.hca import dense_layer_tables

    pos = torch.tensor([0, 1, 5, 7, 8, 4095])
    for cp in (1, 2, 4, 8):
        total = torch.zeros_like(pos)
        for r in range(cp):
            n = causal_local_lens(pos, cp, r)
            want = torch.tensor([len([t for t in range(int(p) + 1) if t % cp == r]) for p in pos])
            assert n.tolist() == want.tolist(), (cp, r)
            total += n
        assert total.tolist() == (pos + 1).tolist()      # every visible token is on exactly one rank
    pt, kv = dense_layer_tables(torch.tensor([33, 16, 0], dtype=torch.int32), torch.tensor([10, 0, 7], dtype=torch.int32), 16)
    assert pt.tolist() == [[10, 11, 12], [0, 0, 0], [0, 0, 0]] and kv.tolist() == [161, 144, 128]


def test_task_offsets_of_a_packed_row():
    """The dynamic scheduler's task index: offsets of the entries of a one-queue schedule, in dependency order."""
    from mega_dsa_cp_b200.layer import build_layer_dag
    from mega_dsa_cp_b200.schedule.codegen import codegen_schedule, pack_queues
    from mega_dsa_cp_b200.schedule.device import task_offsets

    tasks, events, ops = build_layer_dag(3, 4, 2, 128, 2, 1, qpath=True, cand_direct=True)
    s = codegen_schedule(tasks, events, rank=1, n_ctas=1, world_size=2, op_of=ops)
    flat, row = pack_queues(s)
    offs = task_offsets(flat[:row])
    assert len(offs) == len(s.topo) == sum(1 for t in tasks if t.rank == 1)
    assert offs[0] == 0 and all(b - a >= 4 for a, b in zip(offs, offs[1:]))
    assert [flat[o] & 0xFF for o in offs] == [s.op_of[i] for i in s.topo]


def test_ctypes_mirrors_match_the_header_layout(tmp_path):
    """include/mdc.h compiled as plain C by gcc: size of every parameter struct and the offset of every field
    against the ctypes mirrors of _native.py (a mismatch would hand the kernels shifted pointers)."""
    import ctypes as C
    import shutil
    import subprocess

    from mega_dsa_cp_b200 import _native as N

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    pairs = {"mdc_logits_params": N.LogitsParams, "mdc_merge_topk_params": N.MergeTopkParams,
             "mdc_lse_merge_params": N.LseMergeParams, "mdc_sparse_mla_params": N.SparseMlaParams,
             "mdc_event_set": N.EventSetC, "mdc_peer_buffer": N.PeerBufferC, "mdc_compress_params": N.CompressParams,
             "mdc_pingpong_params": N.PingpongParams, "mdc_layer_params": N.LayerParams, "mdc_mega_params": N.MegaParams}
    lines = ["#include <stdio.h>", "#include <stddef.h>", '#include "mdc.h"', "int main(void) {"]
    for cname, mirror in pairs.items():
        lines.append(f'  printf("{cname} %zu\\n", sizeof({cname}));')
        for fname, _ in mirror._fields_:
            lines.append(f'  printf("{cname}.{fname} %zu\\n", offsetof({cname}, {fname}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([gcc, "-std=c99", "-I", os.path.join(root, "include"), str(src), "-o", str(exe)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    got = dict(line.split() for line in subprocess.run([str(exe)], capture_output=True, text=True).stdout.splitlines())
    for cname, mirror in pairs.items():
        assert int(got[cname]) == C.sizeof(mirror), (cname, got[cname], C.sizeof(mirror))
        for fname, _ in mirror._fields_:
            assert int(got[f"{cname}.{fname}"]) == getattr(mirror, fname).offset, (cname, fname)
