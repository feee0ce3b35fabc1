"""The word tokenizer of the host code (host/words.c) against the reference preprocessor: the
committed goldens (made by the reference's own stand-alone tool, tests/golden/make_words_golden.py),
the tool itself where oracle/_ref holds it, and the dictionary's trip through the container."""
import os
import subprocess

import numpy as np
import pytest

from conftest import GOLDEN_DIR

WORD_GOLDENS = sorted(f[6:-4] for f in os.listdir(GOLDEN_DIR) if f.startswith("words_") and f.endswith(".npz"))


def _golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, f"words_{name}.npz"))
    return z, z["text"].tobytes(), int(z["n_words"]), int(z["min_freq"])


@pytest.mark.parametrize("name", [n for n in WORD_GOLDENS if n != "no_return"])
def test_encoder_makes_the_reference_dictionary_and_symbols(pkg, name):
    z, text, n_words, min_freq = _golden(name)
    d, s, n_entries = pkg.host.words_encode(text, n_words, min_freq)
    assert d == z["dict"].tobytes()
    assert np.array_equal(s, z["symbols"])
    assert n_entries == pkg.host.words_count(d) == d.count(b"\n") >= 256


@pytest.mark.parametrize("name", [n for n in WORD_GOLDENS if n != "no_return"])
def test_decoder_reads_the_reference_files(pkg, name):
    z, text, _, _ = _golden(name)
    assert pkg.host.words_decode(z["dict"].tobytes(), z["symbols"]) == text


def test_encoder_returns_where_the_reference_loops_forever(pkg):
    """Two words that put each other out of use in turn: the reference's loop never ends on this
    text; the state repeats, the encoder here stops there, and what it made decodes."""
    _, text, n_words, min_freq = _golden("no_return")
    d, s, n_entries = pkg.host.words_encode(text, n_words, min_freq)
    assert n_entries > 256 and s.size < len(text)
    assert pkg.host.words_decode(d, s) == text


def test_decoder_errors(pkg):
    H = pkg.host
    d, s, n = H.words_encode(b"hello hello world", 300, 1)
    with pytest.raises(ValueError):
        H.words_decode(d, np.array([n], np.uint16))          # a symbol past the dictionary
    with pytest.raises(ValueError):
        H.words_decode(b"a\n\\x\n", np.array([0], np.uint16))  # an escape that is neither \n nor \\
    # an unterminated last line and empty lines are not entries (preprocess.c:1238-1246)
    assert H.words_count(b"a\n\nb\nc") == 2
    # an entry above 4096 bytes, which the reference's decoder refuses, decodes
    long_entry = b"x" * 5000 + b"\n"
    assert H.words_decode(long_entry, np.array([0, 0], np.uint16)) == b"x" * 10000
    with pytest.raises(ValueError):
        H.words_encode(b"abc", 70000, 1)


def _texts():
    rng = np.random.default_rng(12)
    words = [bytes(rng.integers(97, 123, rng.integers(1, 8)).astype(np.uint8)) for _ in range(60)]
    toks = []
    for i in rng.integers(0, 60, 3000):
        r = rng.random()
        toks.append(words[i].upper() if r < 0.05 else words[i].capitalize() if r < 0.2 else words[i])
        toks.append([b" ", b" ", b", ", b".\n", b"  ", b"(", b")", b""][rng.integers(0, 8)])
    yield b"".join(toks), 700, 2
    yield bytes(rng.integers(0, 256, 4000).astype(np.uint8)), 1000, 2
    yield bytes(rng.integers(0, 6, 3000).astype(np.uint8)), 400, 3
    yield b"ab" * 3000, 300, 1
    yield b"The Quick BROWN fox. " * 200, 256, 1
    yield b"The Quick BROWN fox. " * 200, 257, 0


def test_encoder_and_decoder_against_the_reference_tool(pkg, oracle, tmp_path):
    """Live comparison with the reference's stand-alone preprocessor, both directions."""
    exe = oracle.preprocess_ref()
    if exe is None:
        pytest.skip("oracle/_ref/preprocess_ref is not built (no reference tree)")
    f = {k: str(tmp_path / k) for k in ("in", "dict", "sym", "out")}
    compared = 0
    for text, n_words, min_freq in _texts():
        open(f["in"], "wb").write(text)
        d, s, _ = pkg.host.words_encode(text, n_words, min_freq)
        try:
            subprocess.run([exe, "c", f["dict"], f["in"], f["sym"], str(n_words), str(min_freq)], check=True,
                           capture_output=True, timeout=10)
            assert d == open(f["dict"], "rb").read()
            assert s.astype(">u2").tobytes() == open(f["sym"], "rb").read()
            compared += 1
        except subprocess.TimeoutExpired:   # the reference's loop does not end on this text: decode only
            open(f["dict"], "wb").write(d)
            open(f["sym"], "wb").write(s.astype(">u2").tobytes())
        subprocess.run([exe, "d", f["dict"], f["sym"], f["out"]], check=True, capture_output=True, timeout=60)
        assert open(f["out"], "rb").read() == text == pkg.host.words_decode(d, s)
    assert compared >= 5


def test_dictionary_rides_in_the_container(pkg, oracle):
    """Text -> words -> nch_compress with the dictionary in the header -> nch_decompress -> text, the
    model being the CPU oracle; the header layout is flag, two sizes, a zlib stream (nncp.c:3222-3261)."""
    import zlib
    from test_host_code import _oracle_ops
    H = pkg.host
    _, text, _, _ = _golden("prose_small_dict")
    text = text[:1500]
    d, s, n_entries = H.words_encode(text, 300, 3)
    p = pkg.abi.make_params(n_layer=1, d_model=32, n_head=2, d_key=16, d_inner=64, d_pos=16, mem_len=16,
                            seg_len=16, n_streams=4, n_symbols=H.alphabet_size(n_entries), init_range=0.1,
                            lr=1e-2)
    fp = H.file_params(p, block_len=256, dictionary=d)
    data, _ = H.compress(_oracle_ops(pkg, oracle.OracleModel(p)), fp, s, H.EVAL_SEGMENT, H.OUT_FLOAT)

    plain = H.header_bytes(H.file_params(p, block_len=256), s.size)
    at = len(plain) - 5                               # the flag byte sits before the 4-byte symbol count
    assert data[:at] == plain[:at] and plain[at] == 0 and data[at] == 1
    raw_len, z_len = int.from_bytes(data[at + 1:at + 5], "big"), int.from_bytes(data[at + 5:at + 9], "big")
    assert raw_len == len(d) and zlib.decompress(data[at + 9:at + 9 + z_len]) == d
    assert data[at + 9:at + 9 + z_len] == zlib.compress(d, 9)

    fp2, n_sym, used = H.read_header(data)
    assert fp2.dict_len == len(d) and n_sym == s.size and used == at + 9 + z_len + 4
    assert H.read_dict(data) == d and H.read_dict(plain) is None
    back = H.decompress(_oracle_ops(pkg, oracle.OracleModel(p)), data, H.OUT_FLOAT)
    assert np.array_equal(back, s)
    assert H.words_decode(H.read_dict(data), back) == text
    with pytest.raises(ValueError):
        H.read_dict(data[:at + 20])                   # cut inside the zlib stream


def test_text_level_calls_round_trip(pkg, oracle):
    """compress_text / decompress_text: text in, file with its dictionary out, text back; the model
    (here the CPU oracle behind the plugin table) is sized from the dictionary and rebuilt from the header."""
    from test_host_code import _oracle_ops
    H = pkg.host
    _, text, _, _ = _golden("prose_small_dict")
    text = text[:1200]
    base = pkg.abi.make_params(n_layer=1, d_model=32, n_head=2, d_key=16, d_inner=64, d_pos=16, mem_len=16,
                               seg_len=16, n_streams=4, init_range=0.1, lr=1e-2)
    made = []

    def bind(p):
        made.append(p.n_symbols)
        return _oracle_ops(pkg, oracle.OracleModel(p))

    data, st = H.compress_text(text, 300, 3, base, bind=bind, unbind=lambda ops: None, block_len=256)
    assert st.n_symbols < len(text) and made[0] % 8 == 0 and made[0] > 256
    assert H.decompress_text(data, bind=bind, unbind=lambda ops: None) == text
    assert made[1] == made[0]
    padded, _ = H.compress_text(text, 300, 3, base, bind=bind, unbind=lambda ops: None, block_len=256,
                                pad_alphabet=True)
    assert made[-1] == 512 and H.decompress_text(padded, bind=bind, unbind=lambda ops: None) == text
    # a file without a dictionary holds bytes
    raw = np.frombuffer(text[:300], np.uint8).astype(np.uint16)
    p = base.copy(n_symbols=256)
    plain, _ = H.compress(bind(p), H.file_params(p, block_len=256), raw, H.EVAL_SEGMENT, H.OUT_FLOAT)
    assert H.decompress_text(plain, bind=bind, unbind=lambda ops: None) == text[:300]
