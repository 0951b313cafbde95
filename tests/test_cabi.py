"""CPU: the C-ABI library builds, loads and exports exactly what include/flexsae_b200.h declares,
the ctypes signatures agree with the header, and argument checks that need no GPU work."""
import ctypes
import os
import re

from flexsae_b200 import _native as nv

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_prototypes():
    text = open(os.path.join(ROOT, "include", "flexsae_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"#ifdef FLEXSAE_TRACE.*?#endif", "", text, flags=re.S)    # tuning builds only: not in the default library
    protos = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(flexsae_\w+)\s*\(([^;{]*?)\)\s*;", text):
        args = m.group(3).strip()
        n = 0 if args in ("", "void") else len(args.split(","))
        protos[m.group(2)] = (n, args)
    return protos


def test_library_exports_every_declared_symbol():
    lib = nv.load()
    protos = header_prototypes()
    assert len(protos) >= 9
    for name in protos:
        assert hasattr(lib, name), name


def test_ctypes_signatures_match_header():
    protos = header_prototypes()
    assert set(protos) == set(nv.SIGNATURES)
    for name, (n, args) in protos.items():
        res, argtypes = nv.SIGNATURES[name]
        assert len(argtypes) == n, (name, n, len(argtypes))
        for decl, ct in zip(args.split(",") if n else [], argtypes):
            decl = decl.strip()
            if "*" in decl and "char" not in decl:
                assert ct is ctypes.c_void_p, (name, decl)
            elif decl.startswith("int64_t"):
                assert ct is ctypes.c_int64, (name, decl)
            elif decl.startswith("size_t"):
                assert ct is ctypes.c_size_t, (name, decl)
            elif decl.startswith("double"):
                assert ct is ctypes.c_double, (name, decl)
            elif decl.startswith("int "):
                assert ct is ctypes.c_int, (name, decl)


def test_options_and_workspace_sizes_without_gpu():
    lib = nv.load()
    assert lib.flexsae_version() >= 100
    nv.set_option("lanes_bwd", 16)
    assert nv.get_option("lanes_bwd") == 16
    nv.set_option("lanes_bwd", 0)
    assert lib.flexsae_set_option(b"lanes_bwd", 5) != 0 and b"lanes_bwd" in lib.flexsae_last_error()
    assert lib.flexsae_set_option(b"no_such_option", 1) != 0
    # headline shape: two [F, 256] fp32 slabs + per-piece dvals partials + dbias partial rows
    nv.set_option("lanes_bwd", 32)
    n = lib.flexsae_bwd_workspace_bytes(nv.HIER, 4096, 128, 65536, 2304, nv.BF16, nv.DW_ATOMIC)
    nv.set_option("lanes_bwd", 0)
    assert 2 * 65536 * 256 * 4 <= n <= 2 * 65536 * 256 * 4 + 9 * 4096 * 128 * 4 + 4096 * 2304 * 4 + 512 * 2304 * 4 + 8192
    assert lib.flexsae_fwd_workspace_bytes(nv.HIER, 4096, 128, 65536, 2304, nv.BF16) >= 9 * 4096 * 4
    # rejected shapes give 0 and an explanation
    assert lib.flexsae_fwd_workspace_bytes(nv.HIER, 4096, 128, 65536, 2301, nv.BF16) == 0
    assert b"multiple" in lib.flexsae_last_error()
    assert lib.flexsae_fwd_workspace_bytes(7, 1, 1, 1, 8, nv.BF16) == 0


def test_null_pointers_are_rejected_before_any_launch():
    lib = nv.load()
    rc = lib.flexsae_loss_fwd(nv.HIER, None, None, None, None, None, None, None, 1, None, 0, 4, 4, 16, 256,
                              nv.F32, nv.F32, nv.F32, nv.F32, 0.0, None, None)
    assert rc == -1 and b"null" in lib.flexsae_last_error()
    rc = lib.flexsae_loss_bwd(nv.HIER, None, None, None, None, 1, None, None, None, None, None, 0, 4, 4, 16, 256,
                              nv.F32, nv.F32, nv.F32, 0.0, nv.DW_ATOMIC, None, None)
    assert rc == -1
    # a segment count that is not a layout of K is refused (K=4 only has the one-segment layout)
    rc = lib.flexsae_loss_fwd(nv.HIER, None, None, None, None, None, None, None, 3, None, 0, 4, 4, 16, 256,
                              nv.F32, nv.F32, nv.F32, nv.F32, 0.0, None, None)
    assert rc == -1 and b"segments" in lib.flexsae_last_error()


def test_segment_layouts():
    lib = nv.load()
    nv.set_option("segments", 0)
    # small batch: several segments so that one column piece fills the GPU; large batch: one
    assert lib.flexsae_choose_segments(nv.HIER, 4096, 128, 65536, 2304, nv.BF16) >= 2
    assert lib.flexsae_choose_segments(nv.HIER, 65536, 128, 131072, 4096, nv.BF16) == 1
    assert lib.flexsae_choose_segments(nv.HIER, 8, 4, 16, 256, nv.F32) == 1      # K < 8: one segment
    for K in (1, 8, 9, 100, 128, 300):
        ns = lib.flexsae_choose_segments(nv.HIER, 64, K, 1024, 512, nv.F32)
        assert 1 <= ns <= max(1, (K + 7) // 8)
    assert lib.flexsae_state_bytes(nv.HIER, 10, 16, 256, 2) == 2 * 2 * 10 * 256 * 4
    assert lib.flexsae_state_bytes(nv.HIER, 10, 16, 256, 1) == 10 * 256 * 4
    assert lib.flexsae_state_bytes(nv.TOPK, 10, 16, 256, 2) == 10 * 256 * 4


def test_sharded_entry_rejects_bad_arguments_without_a_gpu():
    lib = nv.load()
    three = (ctypes.c_void_p * 3)(16, 32, 48)
    base = [nv.HIER] + [None] * 4 + [1] + [None] * 5 + [0, 4, 4, 16, 256, nv.F32, nv.F32, nv.F32, 0.0, None, None]
    assert lib.flexsae_loss_bwd_sharded(*base, 1, 0, 1, three, three, three, None, None, None) == -1      # world < 2
    assert b"world size" in lib.flexsae_last_error()
    assert lib.flexsae_loss_bwd_sharded(*base, 9, 0, 1, three, three, three, None, None, None) == -1      # world > 8
    assert lib.flexsae_loss_bwd_sharded(*base, 3, 3, 1, three, three, three, None, None, None) == -1      # rank out of range
    assert lib.flexsae_loss_bwd_sharded(*base, 3, 0, 0, three, three, three, None, None, None) == -1      # seq_base < 1
    assert lib.flexsae_loss_bwd_sharded(*base, 3, 0, 1, None, three, three, None, None, None) == -1       # missing buffers
    assert lib.flexsae_loss_bwd_sharded(*base, 3, 0, 1, three, three, three, 64, None, None) == -1        # one multicast address only
    assert lib.flexsae_loss_bwd_sharded(*base, 3, 0, 1, three, three, three, 64, 64, three) == -1    # in place + multicast
    assert lib.flexsae_loss_bwd_sharded(*base, 3, 0, 1, three, three, three, None, None, three) == -1  # [rank] is not dweight
    assert b"dweight_ptrs[rank]" in lib.flexsae_last_error()
    x, y, f = ctypes.c_size_t(), ctypes.c_size_t(), ctypes.c_size_t()
    nv.set_option("lanes_bwd", 16)
    assert lib.flexsae_shard_buffer_bytes(65536, 2304, nv.BF16, 8, ctypes.byref(x), ctypes.byref(y), ctypes.byref(f)) == 0
    nv.set_option("lanes_bwd", 0)
    assert x.value == 2 * 65536 * 128 * 2 and y.value == x.value and f.value >= 8 * 4
    nv.set_option("lanes_bwd", 16)
    assert lib.flexsae_shard_slots(65536, 2304, nv.BF16) == 18 + 5      # pieces + the most draining slots any lag needs
    nv.set_option("lanes_bwd", 0)


def test_small_allreduce_rejects_bad_arguments_without_a_gpu():
    lib = nv.load()
    two = (ctypes.c_void_p * 2)(256, 512)
    n = ctypes.c_size_t()
    assert lib.flexsae_small_allreduce_bytes(8, 16384, ctypes.byref(n)) == 0
    assert n.value == 256 + 2 * 8 * 16384 * 4
    assert lib.flexsae_small_allreduce_bytes(1, 16, ctypes.byref(n)) == -1
    assert lib.flexsae_small_allreduce_bytes(2, 0, ctypes.byref(n)) == -1
    ok = dict(n=4, dtype=nv.F32, world=2, rank=0, seq=1, cap=16)

    def call(**kw):
        a = {**ok, **kw}
        return lib.flexsae_small_allreduce(kw.get("src", 64), 64, a["n"], a["dtype"], a["world"], a["rank"], a["seq"],
                                           kw.get("bufs", two), a["cap"], None, None)

    assert call(world=1) == -1 and b"world size" in lib.flexsae_last_error()
    assert call(world=9) == -1
    assert call(rank=2) == -1
    assert call(n=0) == -1 and call(n=17) == -1 and b"capacity" in lib.flexsae_last_error()
    assert call(dtype=7) == -1
    assert call(seq=0) == -1
    assert call(src=None) == -1 and call(bufs=None) == -1
    assert call(bufs=(ctypes.c_void_p * 2)(256, 0)) == -1 and b"rank 1" in lib.flexsae_last_error()


def test_wait_limit_option_is_validated():
    lib = nv.load()
    before = nv.get_option("wait_limit_ms")
    assert before >= 1000                                # production default: seconds, not a poll count
    assert lib.flexsae_set_option(b"wait_limit_ms", 0) == -1
    assert lib.flexsae_set_option(b"wait_limit_ms", 10 ** 9) == -1
    nv.set_option("wait_limit_ms", 250)
    assert nv.get_option("wait_limit_ms") == 250
    nv.set_option("wait_limit_ms", before)


def test_decoder_of_64_gib_or_more_is_refused():
    """Row-piece offsets are 32-bit counts of 16-byte units: a decoder whose bytes do not fit is refused
    instead of being addressed modulo 2^36."""
    lib = nv.load()
    assert lib.flexsae_fwd_workspace_bytes(nv.HIER, 64, 8, 1 << 21, 16384, nv.BF16) == 0      # exactly 64 GiB
    assert b"64 GiB" in lib.flexsae_last_error()
    assert lib.flexsae_fwd_workspace_bytes(nv.HIER, 64, 8, 1 << 21, 16384 - 8, nv.BF16) > 0
    assert lib.flexsae_choose_segments(nv.HIER, 64, 8, 1 << 22, 4096, nv.F32) == 0           # 64 GiB in fp32
    rc = lib.flexsae_loss_bwd(nv.HIER, None, None, None, None, 1, None, None, None, None, None, 0, 64, 8, 1 << 21, 16384,
                              nv.BF16, nv.F32, nv.BF16, 0.0, nv.DW_ATOMIC, None, None)
    assert rc == -3


def test_sort_entry_rejects_bad_arguments_without_a_gpu():
    lib = nv.load()
    need = lib.flexsae_sort_workspace_bytes(1000, 64)
    assert need >= 5 * 1000 * 4 + 3 * 65 * 4
    assert lib.flexsae_sort_workspace_bytes(0, 64) == 0 and lib.flexsae_sort_workspace_bytes(10, 0) == 0

    def call(idx=64, n=1000, F=64, ws=256, ws_bytes=need):
        return lib.flexsae_sort_by_decoder_row(idx, n, F, ws, ws_bytes, None, None, None, None, None)

    assert call(n=0) == -1 and call(F=0) == -1
    assert call(idx=None) == -1 and call(ws=None) == -1 and b"null" in lib.flexsae_last_error()
    assert call(ws=264) == -1 and b"aligned" in lib.flexsae_last_error()
    assert call(ws_bytes=need - 1) == -2 and b"too small" in lib.flexsae_last_error()


def test_index_skew_entry_and_wide_mode_without_a_gpu():
    """Argument checks of flexsae_index_skew, and the workspace of the wide-piece backward: 32 lanes
    (two 67 MB slabs at the headline shape) unless `lanes_bwd` fixes the width."""
    lib = nv.load()
    assert lib.flexsae_index_skew_workspace_bytes(65536) >= 65536 * 4
    assert lib.flexsae_index_skew_workspace_bytes(0) == 0

    def call(idx=64, B=8, K=4, F=64, ws=256, ws_bytes=256, res=512):
        return lib.flexsae_index_skew(idx, B, K, F, ws, ws_bytes, res, None)

    assert call(B=0) == -1 and call(K=0) == -1 and call(F=0) == -1
    assert call(idx=None) == -1 and call(ws=None) == -1 and call(res=None) == -1
    assert call(ws_bytes=255) == -2 and b"too small" in lib.flexsae_last_error()

    nv.set_option("lanes_bwd", 0)
    shape = (nv.HIER, 8192, 128, 65536, 2304, nv.BF16)
    normal = lib.flexsae_bwd_workspace_bytes(*shape, nv.DW_ATOMIC)            # 16 lanes at this batch size
    wide = lib.flexsae_bwd_workspace_bytes(*shape, nv.DW_ATOMIC_WIDE)
    # two slabs of 256 instead of 128 columns (+67 MB), nine instead of 18 pieces of dvals partials (-38 MB)
    assert abs((wide - normal) - (2 * 65536 * 128 * 4 - 9 * 8192 * 128 * 4)) < 4096     # counters, alignment
    nv.set_option("lanes_bwd", 8)
    try:
        assert lib.flexsae_bwd_workspace_bytes(*shape, nv.DW_ATOMIC_WIDE) == lib.flexsae_bwd_workspace_bytes(*shape, nv.DW_ATOMIC)
    finally:
        nv.set_option("lanes_bwd", 0)
    assert lib.flexsae_bwd_workspace_bytes(*shape, 7) == 0


def test_sharded_backward_plans_wider_pieces_than_the_single_gpu_backward():
    """The batch-sharded backward has its own lane-width rule (and its own workspace size, asked for
    with FLEXSAE_DW_ATOMIC_SHARDED); `lanes_sharded` overrides it."""
    lib = nv.load()
    for name in ("lanes_bwd", "lanes_sharded"):
        nv.set_option(name, 0)
    shape = (65536, 2304, nv.BF16)
    assert lib.flexsae_shard_slots(*shape) == 18 + 5                      # 16 lanes: 18 pieces of 128 columns
    single = lib.flexsae_bwd_workspace_bytes(nv.HIER, 4096, 128, *shape, nv.DW_ATOMIC)
    sharded = lib.flexsae_bwd_workspace_bytes(nv.HIER, 4096, 128, *shape, nv.DW_ATOMIC_SHARDED)
    nv.set_option("lanes_bwd", 16)
    forced16 = lib.flexsae_bwd_workspace_bytes(nv.HIER, 4096, 128, *shape, nv.DW_ATOMIC)
    nv.set_option("lanes_bwd", 8)
    forced8 = lib.flexsae_bwd_workspace_bytes(nv.HIER, 4096, 128, *shape, nv.DW_ATOMIC)
    nv.set_option("lanes_bwd", 0)
    # one GPU, 8 contributions per decoder row (B*K = 8*F): 8 lanes, whose slabs stay in L2; sharded: 16
    assert single == forced8 and sharded == forced16 and forced16 != forced8 and min(forced8, forced16) > 0
    # above 8 contributions per decoder row the single-GPU backward takes 16 lanes as well
    nv.set_option("lanes_bwd", 16)
    dense16 = lib.flexsae_bwd_workspace_bytes(nv.HIER, 4097, 128, *shape, nv.DW_ATOMIC)
    nv.set_option("lanes_bwd", 0)
    assert lib.flexsae_bwd_workspace_bytes(nv.HIER, 4097, 128, *shape, nv.DW_ATOMIC) == dense16
    nv.set_option("lanes_sharded", 8)
    assert lib.flexsae_shard_slots(*shape) == 36 + 5
    nv.set_option("lanes_sharded", 0)
    nv.set_option("lanes_bwd", 32)                                         # a forced backward width applies to both
    assert lib.flexsae_shard_slots(*shape) == 9 + 5
    nv.set_option("lanes_bwd", 0)
    assert lib.flexsae_bwd_workspace_bytes(nv.HIER, 4096, 128, *shape, 7) == 0
