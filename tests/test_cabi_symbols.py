"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "dmlx_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    from dmlx_b200 import _lib

    names = declared_functions()
    assert len(names) > 60
    missing = [n for n in names if not hasattr(_lib.lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_status_names_and_version():
    from dmlx_b200 import _lib

    assert _lib.lib.b200_version() >= 100
    assert _lib.lib.b200_status_name(1) == b"InsufficientBlocks"
    assert _lib.lib.b200_status_name(2) == b"InvalidBlockId"
    assert _lib.lib.b200_status_name(5) == b"InvalidBatchIndex"


def test_compute_fails_loudly_without_a_gpu():
    """No CPU fallback: on a machine without a CUDA device the compute entry points return NoDevice."""
    import torch

    from dmlx_b200 import _lib

    if torch.cuda.is_available():
        return
    assert _lib.lib.b200_device_available() == 0
    cfg = _lib.KvConfig(1, 2, 64, 32, 8, 2, 4, 0, 16, 8, 0)
    h = ctypes.c_void_p()
    assert _lib.lib.b200_kv_create(ctypes.byref(cfg), ctypes.byref(h)) == _lib.ERR_NO_DEVICE
    assert b"no CPU fallback" in _lib.lib.b200_last_error()


def test_struct_layouts_match_the_header(tmp_path):
    """The ctypes mirrors of the header's structs have the header's sizes and field offsets (the header compiled
    as C99 by gcc prints them)."""
    import shutil
    import subprocess

    from dmlx_b200 import _lib

    if shutil.which("gcc") is None:
        return
    pairs = {
        "b200_pack_desc": _lib.PackDesc, "b200_token_output": _lib.TokenOutput, "b200_sample_params": _lib.SampleParams,
        "b200_kv_config": _lib.KvConfig, "b200_llama_config": _lib.LlamaConfig, "b200_qmm_partials": _lib.QmmPartials,
        "b200_moe_config": _lib.MoeConfig, "b200_ep_watch_ops": _lib.EpWatchOps,
    }
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "dmlx_b200.h"', 'int main(void) {']
    for cname, cls in pairs.items():
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for fname, _ in cls._fields_:
            lines.append(f'  printf("{cname} {fname} %zu\\n", offsetof({cname}, {fname}));')
    lines += ['  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    seen = 0
    for line in out:
        if not line:
            continue
        cname, what, value = line.split()
        cls = pairs[cname]
        if what == "size":
            assert ctypes.sizeof(cls) == int(value), (cname, ctypes.sizeof(cls), value)
        else:
            assert getattr(cls, what).offset == int(value), (cname, what, getattr(cls, what).offset, value)
        seen += 1
    assert seen > 40

