"""Host-side checks that need no GPU: the shared library loads, exports every
entry point include/mcep.h declares, computes the buffer size hint like the
reference, and fails loudly (no silent fallback) where a device is needed."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "mcep.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(mcep_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    from mooncake_b200 import build
    lib = ctypes.CDLL(build.build())
    names = _declared_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mcep.h but not exported"


def _reference_hint(M, H, R, E):
    # mooncake-ep/include/mooncake_ep_buffer.h:42-61: two buffers, each with send and
    # receive signals (E ints) and send and receive data (E*M*(2*16 + 2H) bytes)
    sig = E * 4
    data = E * M * (2 * 16 + H * 2)
    return 4 * sig + 4 * data


@pytest.mark.parametrize("M,H,R,E", [(128, 2048, 2, 16), (128, 7168, 8, 256), (4096, 7168, 8, 256),
                                     (256, 4096, 8, 128), (4096, 4096, 8, 8), (1, 128, 1, 1)])
def test_buffer_size_hint_matches_reference_formula(M, H, R, E):
    from mooncake_b200 import Buffer, ep
    assert ep.get_ep_buffer_size_hint(M, H, R, E) == _reference_hint(M, H, R, E)
    assert Buffer.get_ep_buffer_size_hint(M, H, R, E) == _reference_hint(M, H, R, E)


def test_known_sizes():
    from mooncake_b200 import ep
    assert ep.get_ep_buffer_size_hint(128, 7168, 8, 256) == 1883246592       # config 2: 1.88 GB
    assert round(ep.get_ep_buffer_size_hint(4096, 7168, 8, 256) / 1e9, 1) == 60.3  # config 3


def test_module_surface_matches_reference_binding():
    """Names the reference's pybind module and wrapper expose
    (mooncake-ep/src/ep_py.cpp:14-46, mooncake_ep_buffer.py)."""
    from mooncake_b200 import ep, mooncake_ep_buffer
    assert ep.MAX_QP_COUNT == 256
    for m in ("ibgda_disabled", "p2p_enabled", "use_fast_path", "update_local_qpns", "is_roce",
              "sync_ibgda_peers", "get_mr_info", "get_gid", "get_local_qpns", "get_local_lids",
              "get_ipc_handle", "sync_nvlink_ipc_handles", "dispatch", "combine"):
        assert callable(getattr(ep.Buffer, m))
    for m in ("current_stream_wait", "synchronize"):
        assert callable(getattr(ep.EventHandle, m))
    for m in ("connect", "update_ep_member", "get_ep_buffer_size_hint", "dispatch", "combine",
              "get_next_combine_buffer"):
        assert callable(getattr(mooncake_ep_buffer.Buffer, m))
    assert callable(mooncake_ep_buffer.EventOverlap.current_stream_wait)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device behaviour")
def test_no_device_is_a_loud_error_not_a_fallback():
    from mooncake_b200 import ep
    with pytest.raises(RuntimeError, match="CUDA error"):
        ep.Buffer(0, 1, 1 << 20)


def test_zero_copy_surface_exists_and_shapes_the_combine_buffer():
    """`get_next_combine_buffer(handle)` (documented by the reference,
    docs/source/design/mooncake-ep.md:165-167, rejected by its wrapper,
    mooncake_ep_buffer.py:680-681) returns `[E/R, R*M, H]` bf16; where the runtime
    names no symmetric tensor (a single rank) it is an ordinary tensor."""
    import torch
    from mooncake_b200.mooncake_ep_buffer import Buffer

    class _NoSymmetricMemory:
        def next_combine_buffer(self, M, hidden, num_experts):
            return 0, 0

    b = Buffer.__new__(Buffer)
    b.group_size, b.runtime = 2, _NoSymmetricMemory()
    src_info = torch.zeros((4, 2 * 8), dtype=torch.int32)
    t = b.get_next_combine_buffer((src_info, None, 8, 128, 8))
    assert t.shape == (4, 16, 128) and t.dtype == torch.bfloat16


def test_pybind_binding_compiles_and_has_the_reference_module_surface(tmp_path):
    """The compiled alternative to the ctypes binding (what would replace
    mooncake-ep/src/ep_py.cpp): builds against include/mcep.h, links libmcep.so,
    and exposes the names the reference's wrapper uses
    (mooncake-wheel/mooncake/mooncake_ep_buffer.py:108-110, 185-304, 488-507, 641-660)."""
    from tests.pybind_build import build_and_import
    m = build_and_import(str(tmp_path))
    assert m.MAX_QP_COUNT == 256
    assert m.get_ep_buffer_size_hint(128, 7168, 8, 256) == 1883246592
    for name in ("ibgda_disabled", "p2p_enabled", "use_fast_path", "is_roce", "update_local_qpns",
                 "sync_ibgda_peers", "get_mr_info", "get_gid", "get_local_qpns", "get_local_lids",
                 "get_ipc_handle", "sync_nvlink_ipc_handles", "dispatch", "combine"):
        assert hasattr(m.Buffer, name), name
    assert hasattr(m.EventHandle, "current_stream_wait") and hasattr(m.EventHandle, "synchronize")
    # the elastic class of the same module (mooncake-ep/src/ep_py.cpp:48-87)
    for name in ("calculate_buffer_size", "get_physical_domain_size", "get_logical_domain_size",
                 "get_theoretical_num_sms", "ibgda_disabled", "use_fast_path", "update_local_qpns", "is_roce",
                 "sync_ibgda_peers", "get_mr_info", "get_gid", "get_local_qpns", "get_local_lids",
                 "get_ipc_handle", "sync_nvlink_ipc_handles", "dispatch", "combine"):
        assert hasattr(m.ElasticBuffer, name), name
    assert m.calculate_elastic_buffer_size(8, 128, 4096, 8, False, True, True) == \
        m.ElasticBuffer.calculate_buffer_size(8, 128, 4096, 8, False, True, True) == \
        2 * 8 * 128 * (32 + 4 * 4096) + 2 * 8 * 128 * 80
    import torch
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="Failed: CUDA error"):  # loud, no fallback
            m.Buffer(0, 1, 1 << 20)
        with pytest.raises(RuntimeError, match="Failed: CUDA error"):
            m.ElasticBuffer(0, 1, 1 << 20, 128, 4096, 8, False, False, True, True, True, 3, 0, 300, 100)
        with pytest.raises(RuntimeError, match="not built"):
            m.ElasticBuffer(0, 1, 1 << 20, 128, 4096, 8, True, False, True, True, True, 3, 0, 300, 100)


_C_KINDS = {"int32_t": ("i", 4), "int64_t": ("i", 8), "uint64_t": ("u", 8)}


def _header_struct(name):
    """[(field, size in bytes)] of a struct in include/mcep.h, in declaration order."""
    text = open(os.path.join(ROOT, "include", "mcep.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), text, flags=re.S).group(1)
    out = []
    for decl in [d.strip() for d in body.split(";") if d.strip()]:
        m = re.match(r"(const\s+)?(\w+)\s*(\*?)\s*(\w+(?:\s*,\s*\w+)*)$", decl)
        assert m, decl
        ctype, ptr = m.group(2), m.group(3)
        for field in [f.strip() for f in m.group(4).split(",")]:
            out.append((field, 8 if ptr else _C_KINDS[ctype][1]))
    return out


@pytest.mark.parametrize("cname,pyname", [("mcep_dispatch_args", "_DispatchArgs"),
                                          ("mcep_combine_args", "_CombineArgs"),
                                          ("mcep_elastic_dispatch_args", "_ElasticDispatchArgs"),
                                          ("mcep_elastic_combine_args", "_ElasticCombineArgs")])
def test_argument_structs_match_the_header(cname, pyname, tmp_path):
    """The ctypes mirror has the header's fields in the header's order, and the
    offsets a C compiler gives them."""
    from mooncake_b200 import ep
    py = getattr(ep, pyname)
    want = _header_struct(cname)
    got = [(n, ctypes.sizeof(t)) for n, t in py._fields_]
    assert got == want
    src = tmp_path / "offsets.c"
    lines = "\n".join(f'    printf("%zu\\n", offsetof({cname}, {n}));' for n, _ in want)
    src.write_text('#include <stddef.h>\n#include <stdio.h>\n#include "mcep.h"\n'
                   f'int main(void) {{\n{lines}\n    printf("%zu\\n", sizeof({cname}));\n    return 0;\n}}\n')
    exe = tmp_path / "offsets"
    import subprocess
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src)], check=True)
    nums = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True,
                                           text=True).stdout.split()]
    assert nums[:-1] == [getattr(py, n).offset for n, _ in want]
    assert nums[-1] == ctypes.sizeof(py)


def test_every_entry_point_cites_what_it_replaces():
    """Each declaration in the header is preceded by a comment that names the
    reference interface it stands in for, or says that there is none."""
    text = open(os.path.join(ROOT, "include", "mcep.h")).read()
    for name in _declared_functions():
        pos = re.search(r"\b%s\s*\(" % name, re.sub(r"/\*.*?\*/", lambda m: " " * len(m.group(0)),
                                                    text, flags=re.S)).start()
        before = text[:pos]
        # the nearest section or declaration comment above the declaration
        # (field comments inside the argument structs are short: skip them)
        comments = [c for c in re.findall(r"/\*.*?\*/", before, flags=re.S) if len(c) > 70]
        assert comments, name
        near = " ".join(comments[-3:])
        assert re.search(r"mooncake-[a-z-]+/|no counterpart|No counterpart|not in the reference|"
                         r"Measurement aid|last failure|has launched", near), name


def test_library_is_rebuilt_when_its_sources_change(tmp_path, monkeypatch):
    """The library counts as stale by the CONTENT of its sources (a digest kept
    beside it), not by file times: a copy of the tree keeps no times, and a
    library older than its sources must not be loaded in silence."""
    from mooncake_b200 import build
    assert not build._stale()
    stamp = open(build.STAMP).read()
    monkeypatch.setattr(build, "STAMP", str(tmp_path / "stamp"))
    assert build._stale()                      # no record of what it was built from
    (tmp_path / "stamp").write_text(stamp)
    assert not build._stale()
    (tmp_path / "stamp").write_text("0" * 64)  # built from something else
    assert build._stale()
    monkeypatch.setenv("MCEP_NVCC_FLAGS", "-DSOMETHING")
    (tmp_path / "stamp").write_text(stamp)
    assert build._stale()                      # other compiler flags are other sources


def test_mooncake_checkout_is_found_through_the_environment(tmp_path, monkeypatch):
    from oracle import build as ob
    fake = tmp_path / "tree"
    (fake / "mooncake-ep" / "src").mkdir(parents=True)
    (fake / "mooncake-ep" / "src" / "mooncake_ep_kernel.cu").write_text("// stand-in")
    monkeypatch.setenv("MOONCAKE_SRC", str(fake))
    assert ob.find_mooncake_src() == str(fake)
    monkeypatch.setenv("MOONCAKE_SRC", str(tmp_path / "nowhere"))
    assert ob.find_mooncake_src() != str(tmp_path / "nowhere")


def test_elastic_wrapper_surface_and_loud_failure_without_a_gpu():
    """The elastic wrapper has the reference's names (mooncake-wheel/mooncake/
    mooncake_elastic_buffer.py:84-774), rejects what is not built before touching
    the device, and has no CPU path."""
    import inspect
    import torch
    from mooncake_b200.mooncake_elastic_buffer import ElasticBuffer, EPHandle

    class Solo:
        def rank(self):
            return 0

        def size(self):
            return 1

    sig = inspect.signature(ElasticBuffer.__init__)
    for name in ("group", "num_bytes", "num_max_tokens_per_rank", "hidden", "num_topk", "use_fp8_dispatch",
                 "deterministic", "allow_hybrid_mode", "allow_multiple_reduction", "num_gpu_timeout_secs"):
        assert name in sig.parameters, name
    for name in ("x", "topk_idx", "topk_weights", "num_experts", "num_max_tokens_per_rank", "expert_alignment",
                 "handle", "do_expand", "do_cpu_sync", "num_sms", "async_with_compute_stream"):
        assert name in inspect.signature(ElasticBuffer.dispatch).parameters, name
    for name in ("x", "handle", "topk_weights", "num_sms", "async_with_compute_stream"):
        assert name in inspect.signature(ElasticBuffer.combine).parameters, name
    for name in ("update_ep_member", "destroy", "barrier", "get_buffer_size_hint", "get_theoretical_num_sms",
                 "get_physical_domain_size", "get_logical_domain_size"):
        assert hasattr(ElasticBuffer, name), name
    md = torch.zeros((5, 6), dtype=torch.int32)
    h = EPHandle(False, 8, 1, 16, 4, torch.zeros((3, 4), dtype=torch.int64), [], torch.zeros(1), torch.zeros(8),
                 md, torch.zeros((3, 4)))
    assert h.num_recv_tokens == 5 and h.native_handle is None
    with pytest.raises(NotImplementedError):
        ElasticBuffer(Solo(), use_fp8_dispatch=True)
    with pytest.raises(NotImplementedError):
        ElasticBuffer(Solo(), allow_multiple_reduction=False)
    assert ElasticBuffer.get_buffer_size_hint(Solo(), 128, 4096, 8) == 0
    from mooncake_b200 import ep
    # 2 parities x R*M rows x (32 + 4H) bytes, plus an 80-byte record per row (8K + 4, 16-byte aligned)
    assert ep.elastic_buffer_size_hint(128, 4096, 8, 8) == 2 * 8 * 128 * (32 + 4 * 4096) + 2 * 8 * 128 * 80
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="Failed: CUDA error"):
            ElasticBuffer(Solo(), num_max_tokens_per_rank=16, hidden=256, num_topk=2)
