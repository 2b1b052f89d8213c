"""The C-ABI library loads and exports every symbol include/fold_b200.h
declares (no compute: this runs without a GPU)."""

import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "fold_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fold_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    import __graft_entry__ as ge

    ge.build()
    lib = ctypes.CDLL(os.path.join(ROOT, "fold_attention_b200", "libfold_b200.so"))
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), n


def test_bad_arguments_return_a_status_and_a_message():
    from fold_attention_b200 import _lib

    rc = _lib.lib.fold_bwd_workspace_layout(1, 1, 1, 1, 1, 64, 0, 0, 0, None)
    assert rc == 1
    assert b"null pointer" in _lib.lib.fold_last_error()
    # sizes are computed on the host: no GPU needed
    n = _lib.lib.fold_bwd_workspace_bytes(4, 32, 32, 8192, 4 * 8192, 128, 0, 0, 0)
    assert n >= 4 * 32 * 8192 * 128 * 4
    # a folding plan (MQA cut four heads at a time) adds the int64 dK and dV accumulators and a longer list
    private = _lib.lib.fold_bwd_workspace_bytes(2, 32, 1, 8192, 2 * 8192, 128, 0, 0, 0)
    folded = _lib.lib.fold_bwd_workspace_bytes(2, 32, 1, 8192, 2 * 8192, 128, 0, 4, 0)
    assert folded >= private + 2 * 8 * 2 * 8192 * 128
    assert _lib.lib.fold_bwd_workspace_bytes(2, 32, 1, 8192, 2 * 8192, 128, 0, 5, 0) == 0   # 5 does not divide 32


def test_the_tail_entries_refuse_what_they_cannot_run():
    """Argument checks come before any CUDA call, so they run without a GPU."""
    import fold_attention_b200.decode.launch  # noqa: F401  (registers fold_decode_run_tail)
    from fold_attention_b200 import _lib

    one = ctypes.c_void_p(256)      # never dereferenced: every call below is refused first

    def tail_decode(rank=16, u=one, vr=one, page_size=128, rows=one):
        return _lib.lib.fold_decode_run_tail(one, one, one, one, one, one, one, rows, u, vr, rank, one, one, one, one, None,
                                             2, 8, 2, 128, 4, page_size, 1, 0, 2, 8.0, one, one, one, one, 0, one, one, one, None)

    assert tail_decode(rank=12) == 1 and b"tail rank 12" in _lib.lib.fold_last_error()
    assert tail_decode(rank=-1) == 1
    assert tail_decode(u=None) == 1 and b"rank 16 only" in _lib.lib.fold_last_error()
    assert tail_decode(rank=0) == 1              # rank 0 takes no u and vr
    assert tail_decode(page_size=32) == 1 and b"one row per 64 keys" in _lib.lib.fold_last_error()
    assert tail_decode(rows=None) == 1

    def tail_append(rank=16, page_size=128, back=1, ysum=one):
        return _lib.lib.fold_tail_append(one, 0, 2, 2, 128, one, 4, page_size, one, back, one, one, one, one, one, ysum, one, rank, None)

    assert tail_append(rank=8) == 1 and b"tail rank 8" in _lib.lib.fold_last_error()
    assert tail_append(page_size=96) == 1
    assert tail_append(back=2) == 1
    assert tail_append(ysum=None) == 1 and b"rank 16 needs" in _lib.lib.fold_last_error()


def test_python_signatures_cover_the_header():
    import fold_attention_b200  # noqa: F401  (registers every signature)
    import fold_attention_b200.decode.static_scratch  # noqa: F401
    from fold_attention_b200 import _lib

    assert set(_declared()) <= set(_lib.exported_symbols())


def test_the_product_never_reaches_for_the_oracle_or_scratch():
    """The oracle is test infrastructure: nothing under the package may import, read
    or run it (or a scratch folder), and the package has no CPU fallback to route
    through; bench.py may use it only in its cpu_baseline / reference arm."""
    pkg = os.path.join(ROOT, "fold_attention_b200")
    for dirpath, _, files in os.walk(pkg):
        if os.sep + "build" in dirpath:
            continue
        for f in files:
            if not f.endswith((".py", ".cu", ".cuh", ".h")):
                continue
            text = open(os.path.join(dirpath, f)).read()
            assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), (dirpath, f)
            assert not re.search(r"[\"'/]_work\b", text), (dirpath, f)
    bench = open(os.path.join(ROOT, "bench.py")).read()
    uses = [m.start() for m in re.finditer(r"from oracle import", bench)]
    assert len(uses) == 1 and "def cpu_reference_tflops" in bench[:uses[0]]
    assert bench.rfind("def ", 0, uses[0]) == bench.find("def cpu_reference_tflops")
