"""Writes the tokenizer goldens words_<name>.npz: seeded synthetic text run through the reference's
own stand-alone preprocessor (oracle/_ref/preprocess_ref, built from the reference's preprocess.c
by oracle/Makefile).  Each file holds the text, the dictionary text and the 16-bit symbols the
reference made of it, with the n_words / min_freq it was given.  On the `no_return` text the
reference's dictionary loop never ends (two words put each other out of use in turn); that file
holds the text alone, and the script checks that the reference still runs out of time on it.

    python tests/golden/make_words_golden.py        (needs the reference tree for oracle/_ref)
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def prose(seed, n_tokens, vocab=120):
    """Word soup with capitals, all-caps, punctuation, doubled spaces and line ends."""
    rng = np.random.default_rng(seed)
    words = [bytes(rng.integers(97, 123, rng.integers(1, 9)).astype(np.uint8)) for _ in range(vocab)]
    gaps = [b" ", b" ", b" ", b" ", b", ", b".\n", b"  ", b" (", b") ", b"-", b"", b"; "]
    out = []
    for i in rng.zipf(1.4, n_tokens) % vocab:
        w, r = words[i], rng.random()
        out += [w.capitalize() if r < 0.12 else w.upper() if r < 0.16 else w, gaps[rng.integers(0, len(gaps))]]
    return b"".join(out)


def reserved_and_high(seed, n):
    """Bytes 1..4 (the marker codes), backslashes, line ends and multi-byte characters."""
    rng = np.random.default_rng(seed)
    s = "".join(chr(int(c)) for c in rng.choice([0x61, 0x62, 0xe9, 0x4e2d, 0x20, 0x41, 0x42, 0x0a, 0x3b1, 0x5c,
                                                  1, 2, 3, 4], n))
    return s.encode()


def repeats(seed, n_par, times):
    rng = np.random.default_rng(seed)
    return bytes(rng.integers(32, 127, n_par).astype(np.uint8)) * times


def cycling(seed=386, n=1344):
    rng = np.random.default_rng(seed)
    s = "".join(chr(int(c)) for c in rng.choice([0x61, 0x62, 0xe9, 0x4e2d, 0x20, 0x41, 0x42, 0x0a, 0x3b1], n))
    return s.encode()


NO_RETURN = ("no_return", cycling(), 512, 2)

CASES = {
    "prose": (prose(1, 2500), 512, 2),
    "prose_small_dict": (prose(2, 1500, vocab=40), 300, 5),
    "reserved_high": (reserved_and_high(3, 1500), 400, 2),
    "repeats": (repeats(4, 90, 25), 1000, 1),
    "bytes_only": (prose(5, 300), 256, 2),
    "empty": (b"", 512, 2),
    "one_byte": (b"Q", 512, 2),
}


def main():
    from oracle import oracle as orc
    exe = orc.preprocess_ref()
    if exe is None:
        raise SystemExit("oracle/_ref/preprocess_ref is not built (make -C oracle REF=<reference tree>)")
    with tempfile.TemporaryDirectory() as td:
        for name, (text, n_words, min_freq) in CASES.items():
            f = {k: os.path.join(td, k) for k in ("in", "dict", "sym")}
            open(f["in"], "wb").write(text)
            subprocess.run([exe, "c", f["dict"], f["in"], f["sym"], str(n_words), str(min_freq)], check=True,
                           capture_output=True, timeout=60)
            np.savez_compressed(os.path.join(HERE, f"words_{name}.npz"),
                                text=np.frombuffer(text, np.uint8),
                                dict=np.frombuffer(open(f["dict"], "rb").read(), np.uint8),
                                symbols=np.frombuffer(open(f["sym"], "rb").read(), ">u2").astype(np.uint16),
                                n_words=n_words, min_freq=min_freq)
            print(name, len(text), "bytes ->", os.path.getsize(f["sym"]) // 2, "symbols")
        name, text, n_words, min_freq = NO_RETURN
        open(os.path.join(td, "in"), "wb").write(text)
        try:
            subprocess.run([exe, "c", os.path.join(td, "dict"), os.path.join(td, "in"), os.path.join(td, "sym"),
                            str(n_words), str(min_freq)], capture_output=True, timeout=10)
            raise SystemExit("the reference returned on the no_return text: pick another")
        except subprocess.TimeoutExpired:
            np.savez_compressed(os.path.join(HERE, f"words_{name}.npz"), text=np.frombuffer(text, np.uint8),
                                n_words=n_words, min_freq=min_freq)
            print(name, len(text), "bytes: the reference does not return (10 s)")


if __name__ == "__main__":
    main()
