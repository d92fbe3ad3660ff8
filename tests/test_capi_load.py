"""The C-ABI library builds for sm_100a, loads without a GPU and exports every symbol that
include/rlt_verify.h declares; the host layer refuses CPU tensors instead of falling back."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def library():
    from vllm_rlt_b200 import build

    return ctypes.CDLL(str(build.build()))


def declared_symbols():
    text = (ROOT / "include" / "rlt_verify.h").read_text()
    return sorted(set(re.findall(r"RLT_API[^;(]*?\b(rlt_[a-z_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for required in ("rlt_silu_and_mul", "rlt_kv_write", "rlt_verify_attention", "rlt_accept_greedy",
                     "rlt_accept_rejection", "rlt_rollback", "rlt_argmax_rows", "rlt_sample_rows"):
        assert required in names


def test_library_exports_every_declared_symbol(library):
    for name in declared_symbols():
        assert hasattr(library, name), name


def test_python_binding_covers_every_declared_symbol():
    from vllm_rlt_b200 import _capi

    assert sorted(_capi.SIGNATURES) == declared_symbols()
    lib = _capi.load()
    assert lib.rlt_version().decode().endswith("sm_100a")


def test_workspace_size_is_monotonic_and_aligned(library):
    fn = library.rlt_verify_attention_workspace_bytes
    fn.restype = ctypes.c_size_t
    small = fn(16, 16, 16, 128, 16, 64)
    large = fn(1024, 16, 16, 128, 16, 256)
    assert 0 < small < large and small % 256 == 0 and large % 256 == 0


def test_host_layer_has_no_cpu_fallback():
    import vllm_rlt_b200 as rlt

    with pytest.raises(ValueError, match="CUDA"):
        rlt.silu_and_mul(torch.ones(4), torch.ones(4))
    with pytest.raises(ValueError, match="CUDA"):
        rlt.argmax_rows(torch.ones(2, 8))
    with pytest.raises(ValueError, match="CUDA"):
        rlt.B200PagedAttention()(torch.ones(1, 1, 8), torch.ones(1, 2, 1, 8), torch.ones(1, 2, 1, 8),
                                 torch.zeros(1, 1, dtype=torch.int32), torch.ones(1, dtype=torch.int32))


def test_product_package_never_imports_the_oracle():
    package = ROOT / "vllm_rlt_b200"
    for path in list(package.rglob("*.py")) + list(package.rglob("*.cu")) + list(package.rglob("*.cuh")):
        text = path.read_text()
        for needle in ("import oracle", "from oracle", "librlt_oracle", "orc_", "oracle/"):
            assert needle not in text, (path, needle)


def test_silu_argument_checks_match_the_reference_errors():
    import vllm_rlt_b200 as rlt

    with pytest.raises(ValueError, match="same shape"):
        rlt.silu_and_mul(torch.ones(2, 7), torch.ones(1, 7))
    with pytest.raises(TypeError, match="same dtype"):
        rlt.silu_and_mul(torch.ones(7), torch.ones(7, dtype=torch.float16))
    for dtype in (torch.int32, torch.float64):
        with pytest.raises(TypeError, match="supports float32"):
            rlt.silu_and_mul(torch.ones(7, dtype=dtype), torch.ones(7, dtype=dtype))


def test_header_is_plain_c_and_a_c_program_links_against_the_library(library, tmp_path):
    """The boundary is a C ABI: the header compiles as C99 without CUDA or C++ headers, and a C
    translation unit that takes the address of every entry point links against the library
    (calls that need no GPU run: version string, workspace sizes, argument errors)."""
    import subprocess

    names = declared_symbols()
    source = tmp_path / "abi.c"
    table = ",\n  ".join(f'{{"{n}", (void (*)(void)){n}}}' for n in names)
    source.write_text(f'''
#include <stdio.h>
#include <string.h>
#include "rlt_verify.h"
struct entry {{ const char* name; void (*address)(void); }};
static const struct entry entries[] = {{
  {table}
}};
int main(void) {{
  size_t n = sizeof(entries) / sizeof(entries[0]);
  for (size_t i = 0; i < n; ++i) if (entries[i].address == 0) return 2;
  if (strstr(rlt_version(), "sm_100a") == 0) return 3;
  if (rlt_verify_attention_workspace_bytes(16, 16, 16, 128, 16, 64) == 0) return 4;
  /* invalid arguments come back as a status and a message, never as a crash or an exception */
  if (rlt_silu_and_mul(0, 0, 0, 8, 99, 0) != RLT_ERR_INVALID) return 5;
  if (strlen(rlt_last_error()) == 0) return 6;
  printf("%zu entry points\\n", n);
  return 0;
}}
''')
    binary = tmp_path / "abi"
    lib_dir = ROOT / "vllm_rlt_b200"
    subprocess.run(["/usr/bin/gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", str(ROOT / "include"), str(source),
                    "-o", str(binary), f"-L{lib_dir}", "-lrlt_verify", f"-Wl,-rpath,{lib_dir}"], check=True)
    done = subprocess.run([str(binary)], check=True, capture_output=True, text=True)
    assert done.stdout.strip() == f"{len(names)} entry points"
