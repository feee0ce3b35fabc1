"""The `nncp-metal` front-end (include/nncp_metal_frontend.h): container header, checksum, format
sniffing and the command line of the reference's src/metal/nncp_metal.c, over the GPU compressor.

CPU tests cover the byte layout and the host logic; the GPU tests run the command-line tool end to
end (compress -> decompress must give the input back, byte for byte)."""
import ctypes as C
import os
import struct
import subprocess

import numpy as np
import pytest

from conftest import ROOT

CLI = os.path.join(ROOT, "nncp-metal_b200", "nncp-metal")
HOSTLIB = os.path.join(ROOT, "nncp-metal_b200", "libnncp_host.so")


class Header(C.Structure):
    # NNCPHeader of the reference (src/metal/nncp_metal.c:174-182), field for field
    _fields_ = [("magic", C.c_uint32), ("version", C.c_uint32), ("original_size", C.c_uint32),
                ("compressed_size", C.c_uint32), ("compression_level", C.c_uint16),
                ("quantization_bits", C.c_uint16), ("checksum", C.c_uint32)]


@pytest.fixture(scope="module")
def host(pkg):
    pkg.build_library()
    L = C.CDLL(HOSTLIB)
    L.nncpm_checksum.restype = C.c_uint32
    L.nncpm_checksum.argtypes = [C.c_char_p, C.c_size_t]
    L.nncpm_route.argtypes = [C.POINTER(Header)]
    L.nncpm_estimate_output_size.restype = C.c_size_t
    L.nncpm_estimate_output_size.argtypes = [C.c_size_t]
    L.nncpm_lossless_compress.restype = C.c_size_t
    L.nncpm_lossless_compress.argtypes = [C.c_char_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_int, C.c_char_p]
    L.nncpm_lossless_decompress.restype = C.c_size_t
    L.nncpm_lossless_decompress.argtypes = [C.c_char_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_char_p]
    L.nncpm_last_error.restype = C.c_char_p
    return L


def _text(n, seed):
    rng = np.random.default_rng(seed)
    words = [bytes(rng.integers(97, 123, rng.integers(2, 9)).astype(np.uint8)) for _ in range(80)]
    return b" ".join(words[i] for i in rng.integers(0, 80, n // 3))[:n]


def test_header_is_the_reference_struct(host):
    assert C.sizeof(Header) == 24
    # magic "NNCP" as the reference defines it (0x4E4E4350), native-endian fields
    raw = struct.pack("=IIIIHHI", 0x4E4E4350, 1, 1000, 524, 8, 8, 0xDEADBEEF)
    h = Header.from_buffer_copy(raw)
    assert (h.magic, h.version, h.original_size, h.compressed_size) == (0x4E4E4350, 1, 1000, 524)
    assert (h.compression_level, h.quantization_bits, h.checksum) == (8, 8, 0xDEADBEEF)


def test_checksum_is_the_reference_fold(host):
    rng = np.random.default_rng(1)
    for n in (0, 1, 17, 4096):
        data = rng.integers(0, 256, n, dtype=np.uint8).tobytes()
        c = 0
        for b in data:      # checksum = checksum * 31 + byte (nncp_metal.c:307-311), 32-bit wrap
            c = (c * 31 + b) & 0xFFFFFFFF
        assert host.nncpm_checksum(data, n) == c


def test_decoder_routes_follow_the_reference(host):
    # nncp_metal.c:1277-1282: bit 15 -> Neural Engine; level 6 / 8 with 8 bits -> LSTM / Transformer;
    # other levels <= 9 with 8 bits -> CPU NNCP Original; anything else unknown
    want = {(0x8006, 8): 1, (6, 8): 2, (8, 8): 3, (3, 8): 4, (9, 8): 4, (7, 8): 4, (12, 8): 5, (8, 16): 5}
    for (lvl, bits), route in want.items():
        h = Header(0x4E4E4350, 1, 0, 24, lvl, bits, 0)
        assert host.nncpm_route(C.byref(h)) == route, (lvl, bits)


def test_cli_usage_and_refusals():
    run = lambda *a: subprocess.run([CLI, *a], capture_output=True, text=True, timeout=60)
    r = run("-h")
    assert r.returncode == 0 and "c, compress" in r.stdout and "d, decompress" in r.stdout
    assert run().returncode == 1
    r = run("frobnicate", "a", "b")
    assert r.returncode == 1 and "Unknown command 'frobnicate'" in r.stdout
    r = run("compress", "only_one")
    assert r.returncode == 1 and "compress command requires input and output file arguments" in r.stdout
    r = run("c", "a", "b", "--cpu")
    assert r.returncode == 1 and "no CPU model" in r.stdout
    assert run("neural", "a", "b").returncode == 1
    r = run("test")
    assert r.returncode == 0 and "ABI version 1" in r.stdout


def test_cli_refuses_foreign_and_damaged_files(tmp_path):
    run = lambda *a: subprocess.run([CLI, *a], capture_output=True, text=True, timeout=60)
    short = tmp_path / "short.nncp"
    short.write_bytes(b"NNCP")
    r = run("d", str(short), str(tmp_path / "o"))
    assert r.returncode == 1 and "Cannot read file header" in r.stdout
    lstm = tmp_path / "lstm.nncp"
    lstm.write_bytes(struct.pack("=IIIIHHI", 0x4E4E4350, 1, 10, 34, 6, 8, 0) + b"\0" * 10)
    r = run("d", str(lstm), str(tmp_path / "o"), "-v")   # files first, as the reference parses them
    assert r.returncode == 1 and "Auto-detected compression format: LSTM" in r.stdout
    assert "another codec" in r.stdout
    bad = tmp_path / "bad.nncp"
    bad.write_bytes(struct.pack("=IIIIHHI", 0x12345678, 1, 10, 34, 8, 8, 0) + b"\0" * 10)
    assert run("d", str(bad), str(tmp_path / "o")).returncode == 1
    # an empty file is a header alone and needs no model
    empty, back = tmp_path / "empty.nncp", tmp_path / "empty.out"
    empty.write_bytes(struct.pack("=IIIIHHI", 0x4E4E4350, 1, 0, 24, 8, 8, 0))
    assert run("d", str(empty), str(back)).returncode == 0 and back.read_bytes() == b""


def test_compress_fails_loudly_without_a_gpu(host, tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    out = C.create_string_buffer(4096)
    assert host.nncpm_lossless_compress(b"hello world " * 20, 240, out, 4096, 6, None) == 0
    assert b"no usable B200" in host.nncpm_last_error()
    src = tmp_path / "in.txt"
    src.write_bytes(b"hello world " * 20)
    r = subprocess.run([CLI, "c", str(src), str(tmp_path / "o.nncp")], capture_output=True, text=True, timeout=60)
    assert r.returncode == 1 and "ERROR" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("level,n", [(3, 5000), (6, 9000), (8, 20000)])
def test_cli_round_trip_on_the_gpu(tmp_path, level, n):
    data = _text(n, level)
    src, cmp_, back = tmp_path / "in.txt", tmp_path / "out.nncp", tmp_path / "back.txt"
    src.write_bytes(data)
    r = subprocess.run([CLI, "compress", str(src), str(cmp_), "-l", str(level), "-v"], capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stdout + r.stderr
    blob = cmp_.read_bytes()
    h = Header.from_buffer_copy(blob[:24])
    c = 0
    for b in data:
        c = (c * 31 + b) & 0xFFFFFFFF
    assert (h.magic, h.version, h.original_size, h.compressed_size) == (0x4E4E4350, 1, n, len(blob))
    assert (h.compression_level, h.quantization_bits, h.checksum) == (8, 8, c)
    assert blob[24:28] == bytes.fromhex("b727ac58")       # the nncp.c stream magic opens the payload
    assert len(blob) < 0.95 * n      # it learns something even on a short file (the wide level-8 model slowly)
    r = subprocess.run([CLI, "d", str(cmp_), str(back)], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout + r.stderr
    assert back.read_bytes() == data
    # one flipped payload byte: the decoder notices (checksum) instead of writing wrong data
    dmg = bytearray(blob)
    dmg[len(dmg) // 2] ^= 0x40
    bad = tmp_path / "bad.nncp"
    bad.write_bytes(bytes(dmg))
    r = subprocess.run([CLI, "d", str(bad), str(tmp_path / "bad.out")], capture_output=True, text=True, timeout=900)
    assert r.returncode == 1 and "ERROR" in r.stdout


@pytest.mark.gpu
def test_memory_to_memory_entry_points_on_the_gpu(host):
    data = _text(6000, 11)
    cap = host.nncpm_estimate_output_size(len(data))
    out = C.create_string_buffer(cap)
    n = host.nncpm_lossless_compress(data, len(data), out, cap, 5, None)
    assert n > 24, host.nncpm_last_error()
    back = C.create_string_buffer(len(data))
    m = host.nncpm_lossless_decompress(out.raw[:n], n, back, len(data), None)
    assert m == len(data), host.nncpm_last_error()
    assert back.raw == data
    # a buffer that is too small is reported, not overrun
    assert host.nncpm_lossless_compress(data, len(data), out, 30, 5, None) == 0
    assert b"too small" in host.nncpm_last_error()
