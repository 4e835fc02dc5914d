"""The C-ABI library loads, exports every symbol include/muxb200.h declares, and validates
arguments before touching the GPU (so these checks run without one)."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "muxb200.h").read_text()


def declared_symbols():
    return sorted(set(re.findall(r"\b(mux_[a-z0-9_]+)\s*\(", HEADER)))


def test_header_symbols_exported(built_lib):
    from muxserve_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 30
    raw = C.CDLL(str(_lib.LIB_PATH))
    for n in names:
        assert hasattr(raw, n), f"{n} is declared in include/muxb200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes bindings and header disagree"
    assert built_lib.mux_abi_version() == _lib.ABI_VERSION


def test_struct_sizes_match_header(built_lib):
    """Field-by-field: ctypes layout == what a C compiler makes of the header."""
    import subprocess, tempfile
    from muxserve_b200 import _lib
    src = f'#include <stdio.h>\n#include "{ROOT}/include/muxb200.h"\nint main(){{printf("%zu %zu %zu\\n", ' \
          'sizeof(mux_cache_write_args_t), sizeof(mux_attn_args_t), sizeof(mux_attn_mixed_args_t));return 0;}'
    with tempfile.TemporaryDirectory() as d:
        (Path(d) / "s.c").write_text(src)
        subprocess.run(["gcc", "-o", f"{d}/s", f"{d}/s.c"], check=True)
        sizes = [int(x) for x in subprocess.run([f"{d}/s"], capture_output=True, text=True, check=True).stdout.split()]
    assert sizes == [C.sizeof(_lib.CacheWriteArgs), C.sizeof(_lib.AttnArgs), C.sizeof(_lib.AttnMixedArgs)]


def test_validation_happens_before_any_launch(built_lib):
    from muxserve_b200 import _lib
    L = built_lib
    a = _lib.AttnArgs()
    assert L.mux_paged_attention(None, None, 0, None) == -1
    a.dtype, a.head_size, a.block_size = 7, 128, 16
    assert L.mux_paged_attention(C.byref(a), None, 0, None) == -2          # dtype
    a.dtype, a.head_size = 0, 64
    assert L.mux_paged_attention(C.byref(a), None, 0, None) == -3          # head size
    a.head_size, a.block_size = 128, 24
    assert L.mux_paged_attention(C.byref(a), None, 0, None) == -4          # block size
    a.block_size, a.num_seqs, a.num_q_heads, a.num_kv_heads, a.num_blocks = 16, 4, 12, 5, 64
    assert L.mux_paged_attention(C.byref(a), None, 0, None) == -7          # 12 q heads over 5 kv heads
    a.num_kv_heads = 4
    assert L.mux_paged_attention(C.byref(a), None, 0, None) == -1          # null tensors
    for f in ("out", "q", "key_cache", "value_cache", "block_tables", "context_lens"):
        setattr(a, f, 0x1000)
    a.q = 0x1008
    assert L.mux_paged_attention(C.byref(a), None, 0, None) == -5          # misaligned q
    a.q, a.max_context_len, a.partition_size = 0x1000, 4096, 512
    need = L.mux_paged_attention_workspace_size(C.byref(a))
    partials = (4 * 4) * 8 * 3 * (128 + 2) * 4                              # items x partitions x group x (acc + m,l) fp32
    assert need == partials
    assert L.mux_paged_attention(C.byref(a), None, 0, None) == -8          # workspace missing
    a.partition_size = 100
    assert L.mux_paged_attention(C.byref(a), None, 0, None) == -6          # not a multiple of block_size
    c = _lib.CacheWriteArgs()
    c.dtype, c.head_size, c.block_size, c.num_tokens, c.num_kv_heads, c.num_blocks = 1, 128, 16, 2, 2, 8
    assert L.mux_reshape_and_cache(C.byref(c), None) == -1
    for f in ("k", "v", "key_cache", "value_cache", "slot_mapping"):
        setattr(c, f, 0x2000)
    c.k_token_stride = 12
    assert L.mux_reshape_and_cache(C.byref(c), None) == -5
    m = _lib.AttnMixedArgs()
    m.dtype, m.head_size, m.block_size, m.num_items, m.num_blocks, m.max_group = 0, 128, 16, 3, 8, 9
    assert L.mux_paged_attention_mixed(C.byref(m), None, 0, None) == -7
    assert b"16-byte" in L.mux_strerror(-5)


def test_prefill_validation_and_struct_layout(built_lib):
    import subprocess, tempfile
    from muxserve_b200 import _lib
    L = built_lib
    src = f'#include <stdio.h>\n#include <stddef.h>\n#include "{ROOT}/include/muxb200.h"\nint main(){{printf("%zu %zu %zu\\n", ' \
          'sizeof(mux_prefill_args_t), offsetof(mux_prefill_args_t, cu_seqlens), offsetof(mux_prefill_args_t, key_cache));return 0;}'
    with tempfile.TemporaryDirectory() as d:
        (Path(d) / "s.c").write_text(src)
        subprocess.run(["gcc", "-o", f"{d}/s", f"{d}/s.c"], check=True)
        got = [int(x) for x in subprocess.run([f"{d}/s"], capture_output=True, text=True, check=True).stdout.split()]
    P = _lib.PrefillArgs
    assert got == [C.sizeof(P), P.cu_seqlens.offset, P.key_cache.offset]
    a = P()
    assert L.mux_prefill_attention(None, None) == -1
    a.dtype, a.head_size = 3, 128
    assert L.mux_prefill_attention(C.byref(a), None) == -2                 # dtype
    a.dtype, a.head_size = 1, 96
    assert L.mux_prefill_attention(C.byref(a), None) == -3                 # head size
    a.head_size, a.num_seqs, a.total_tokens, a.max_prompt_len, a.num_q_heads, a.num_kv_heads = 128, 2, 64, 40, 6, 4
    a.scale = 0.1
    assert L.mux_prefill_attention(C.byref(a), None) == -7                 # 6 q heads over 4 kv heads
    a.num_kv_heads, a.scale = 3, 0.0
    assert L.mux_prefill_attention(C.byref(a), None) == -6                 # scale must be positive
    a.scale = 0.1
    assert L.mux_prefill_attention(C.byref(a), None) == -1                 # null tensors
    for f in ("out", "q", "k", "v", "cu_seqlens"):
        setattr(a, f, 0x4000)
    for f in ("out", "q", "k", "v"):
        setattr(a, f + "_seq_stride", 6 * 128)
        setattr(a, f + "_head_stride", 128)
    a.k_head_stride = 100
    assert L.mux_prefill_attention(C.byref(a), None) == -5                 # rows must start on 16-byte boundaries
    a.k_head_stride, a.key_cache, a.block_size = 128, 0x8000, 12
    assert L.mux_prefill_attention(C.byref(a), None) == -4                 # pool block size
    a.block_size = 16
    assert L.mux_prefill_attention(C.byref(a), None) == -1                 # value pool / slots missing
    a.num_seqs = 0
    a.key_cache = None
    assert L.mux_prefill_attention(C.byref(a), None) == 0                  # nothing to do: no launch, no CUDA call


def test_ops_refuse_cpu_tensors(built_lib):
    import torch
    from muxserve_b200 import ops
    kc, vc = torch.zeros(4, 16, 16, 8, dtype=torch.float16), torch.zeros(4, 128, 16, dtype=torch.float16)
    q = torch.zeros(1, 2, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        ops.paged_attention(q, q, kc, vc, None, 1.0, torch.zeros(1, 2, 1, dtype=torch.int32),
                            torch.ones(1, dtype=torch.int32), 16, 1)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from muxserve_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libmuxb200.so")
    with pytest.raises(ImportError, match="no CPU fallback"):
        _lib.lib()


def test_plain_c_client_links_and_runs(built_lib, tmp_path):
    """The header compiles as C and a C program can drive the host side of the library."""
    import subprocess
    from muxserve_b200 import _lib
    exe = tmp_path / "abi_host"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(ROOT / "tests" / "c" / "abi_host.c"),
                    "-o", str(exe), f"-L{_lib.LIB_PATH.parent}", "-lmuxb200", f"-Wl,-rpath,{_lib.LIB_PATH.parent}"],
                   check=True, capture_output=True, text=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and "c abi ok" in out.stdout, out.stdout + out.stderr
