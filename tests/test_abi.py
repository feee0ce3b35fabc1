"""The C-ABI library: loads without a GPU, exports every symbol include/nncu.h declares,
and refuses to work (loudly, with a status code) when there is no device."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "nncu.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nncu_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    pkg.build_library()
    lib = C.CDLL(pkg.loader.LIB)
    names = _declared()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/nncu.h but not exported"
    assert set(names) == set(pkg.abi.PROTOTYPES), "abi.py and include/nncu.h disagree"


def _declared_in(header, prefix):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(" + prefix + r"[a-z0-9_]+)\s*\(", text)))


def test_host_library_exports_every_declared_symbol(pkg):
    """libnncp_host.so carries everything include/nncp_host.h and include/nncp_metal_frontend.h declare
    (typedef names and function-pointer members are not calls: only names followed by an argument list
    at file scope count, which the plugin table's members are not, since they are written (*name))."""
    pkg.build_library()
    lib = C.CDLL(pkg.loader.HOSTLIB)
    host = [n for n in _declared_in("nncp_host.h", "nch_")]
    front = _declared_in("nncp_metal_frontend.h", "nncpm_")
    assert len(host) >= 25 and len(front) >= 10
    for n in host + front:
        assert hasattr(lib, n), f"{n} is declared but not exported by libnncp_host.so"


def test_plugin_table_has_the_layout_of_the_header(pkg):
    """The ctypes mirror of nch_model_ops: one pointer, three ints, then one function pointer per member of
    the header's struct, in the header's order."""
    text = open(os.path.join(ROOT, "include", "nncp_host.h")).read()
    body = text[text.index("typedef struct nch_model_ops {"):text.index("} nch_model_ops;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    members = re.findall(r"\(\*([a-z_0-9]+)\)\(", body)
    fields = [f[0] for f in pkg.host.ModelOps._fields_]
    assert fields[:4] == ["ctx", "n_streams", "seg_len", "n_symbols"]
    assert fields[4:] == members


def test_struct_layout_matches_header(pkg):
    # nncu_params: 12 int32 + 32 int32 + 8 uint8 + 2 float + int32 + uint32 + 4 float + 3 int32
    assert C.sizeof(pkg.abi.Params) == 4 * 12 + 4 * 32 + 8 + 4 * 2 + 4 + 4 + 4 * 4 + 4 * 3
    assert C.sizeof(pkg.abi.AttnShape) == 4 * 11


def test_default_params_and_version(pkg):
    lib = pkg.library()
    assert lib.nncu_abi_version() == 1
    p = pkg.abi.Params()
    lib.nncu_default_params(C.byref(p))
    # the "default" profile of nncp.c:2471-2513
    assert (p.n_layer, p.d_model, p.n_head, p.d_inner, p.seg_len, p.n_streams) == (4, 256, 8, 512, 32, 16)
    assert p.tied_w_r == 1 and p.tied_b_r == 1 and p.ln_flags == pkg.abi.LN_POST


def test_invalid_options_are_rejected_before_any_device_work(pkg):
    lib = pkg.library()
    for over in (dict(d_pos=1000), dict(ln_flags=3), dict(ff_act=4),
                 dict(d_value=7), dict(n_layer=0), dict(n_layer=33)):
        p = pkg.abi.make_params(**over)
        h = C.c_void_p()
        assert lib.nncu_create(C.byref(p), C.byref(h)) == pkg.abi.ERR_INVALID
        assert lib.nncu_last_error() != b""
        assert not h.value


def test_shapes_no_attention_kernel_can_run_are_refused_at_create(pkg):
    """An fp32 model with several hundred keys per row, or a bf16 model with more than 64 queries
    per segment and a long memory, exceeds the shared memory of every attention kernel pair:
    nncu_create says so (NNCU_ERR_RANGE), instead of the first nncu_eval_gradient failing after the
    encoder has already coded a segment."""
    lib = pkg.library()
    for over in (dict(use_bf16=0, mem_len=1024, seg_len=64, d_pos=64),
                 dict(use_bf16=1, mem_len=2048, seg_len=128, d_pos=128, d_key=64)):
        p = pkg.abi.make_params(**over)
        h = C.c_void_p()
        assert lib.nncu_create(C.byref(p), C.byref(h)) == pkg.abi.ERR_RANGE, over
        assert b"shared memory" in lib.nncu_last_error()
        assert not h.value


def test_no_device_means_error_not_fallback(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = pkg.library()
    p = pkg.abi.make_params()
    h = C.c_void_p()
    assert lib.nncu_create(C.byref(p), C.byref(h)) == pkg.abi.ERR_CUDA
    assert b"no CUDA device" in lib.nncu_last_error()
    with pytest.raises(Exception):
        pkg.TrfModel(p)


def test_host_library_serves_a_c_caller(pkg, tmp_path):
    """The header compiled by a C compiler and the library called from C, with no Python between:
    tokenise, write a header that carries the dictionary, read both back, detokenise.  sizeof
    (nch_file_params) seen by C must be the ctypes mirror's."""
    import subprocess
    src = tmp_path / "caller.c"
    src.write_text(r'''
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "nncp_host.h"
int main(void)
{
    const char *text = "The cat sat on the mat. THE CAT sat; the cat sat on the mat again.\n";
    const size_t n = strlen(text);
    uint8_t *dict, *back, *dict2; size_t dict_len, dict2_len, n_sym, back_len; uint16_t *sym; int entries;
    if (nch_words_encode((const uint8_t *)text, n, 300, 2, &dict, &dict_len, &sym, &n_sym, &entries)) return 1;
    nch_file_params fp; memset(&fp, 0, sizeof(fp));
    fp.model.n_layer = 1; fp.model.n_head = 2; fp.model.d_key = 16; fp.model.d_value = 16; fp.model.d_inner = 64;
    fp.model.d_pos = 16; fp.model.mem_len = 16; fp.model.seg_len = 16; fp.model.n_streams = 4;
    fp.model.n_symbols = (entries + 7) & ~7; fp.model.ff_act = NNCU_FF_GELU; fp.model.ln_flags = NNCU_LN_POST;
    fp.lr.val[0] = 1e-3f; fp.block_len.val[0] = 1000.0f;
    fp.dict = dict; fp.dict_len = (uint32_t)dict_len;
    size_t hlen = 0;
    if (nch_write_header(&fp, (uint32_t)n_sym, NULL, 0, &hlen)) return 2;
    uint8_t *h = malloc(hlen);
    if (nch_write_header(&fp, (uint32_t)n_sym, h, hlen, &hlen)) return 3;
    nch_file_params fp2; uint32_t n2; size_t used;
    if (nch_read_header(h, hlen, &fp2, &n2, &used) || used != hlen || n2 != n_sym || fp2.dict_len != dict_len) return 4;
    if (nch_read_dict(h, hlen, &dict2, &dict2_len) || dict2_len != dict_len || memcmp(dict, dict2, dict_len)) return 5;
    if (nch_words_count(dict2, dict2_len) != entries) return 6;
    if (nch_words_decode(dict2, dict2_len, sym, n_sym, &back, &back_len) || back_len != n || memcmp(back, text, n)) return 7;
    printf("%zu %d %zu\n", sizeof(nch_file_params), entries, n_sym);
    nch_free(dict); nch_free(dict2); nch_free(sym); nch_free(back); free(h);
    return 0;
}
''')
    exe = tmp_path / "caller"
    from nncp_metal_b200.loader import HOSTLIB
    r = subprocess.run(["gcc", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src),
                        HOSTLIB, "-Wl,-rpath," + os.path.dirname(HOSTLIB)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, (r.returncode, r.stderr)
    size, entries, n_sym = map(int, r.stdout.split())
    assert size == C.sizeof(pkg.host.FileParams) and entries > 256 and n_sym < 68
