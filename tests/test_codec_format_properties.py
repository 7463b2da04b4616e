"""Property tests of the lossless codec's format (CPU restatement in ``ops/kv_compress.py``): any bit pattern
round-trips, the packed size never exceeds the raw form, the mode byte is one of the three forms, and the
packer really takes the shorter of its two code shapes for the sampled frequencies."""
import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from flexkv_b200.ops import kv_compress as K


def _tile(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.astype(np.uint16).view(np.int16).copy()).view(torch.bfloat16)


@st.composite
def tiles(draw):
    n = draw(st.sampled_from([1024, 2048]))
    kind = draw(st.sampled_from(["normal", "scaled", "bits", "few", "specials"]))
    seed = draw(st.integers(0, 2**31 - 1))
    rng = np.random.default_rng(seed)
    if kind == "normal":
        x = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).to(torch.bfloat16)
        return x.view(torch.int16).numpy().view(np.uint16)
    if kind == "scaled":                                       # channels of very different scales: flat profile
        sc = np.exp2(rng.uniform(-8, 8, size=128)).astype(np.float32)
        x = torch.from_numpy((rng.standard_normal((n // 128, 128)) * sc).astype(np.float32).reshape(-1)).to(torch.bfloat16)
        return x.view(torch.int16).numpy().view(np.uint16)
    if kind == "bits":
        return rng.integers(0, 1 << 16, size=n, dtype=np.uint16)
    if kind == "few":                                          # a handful of distinct values, long runs
        vals = rng.integers(0, 1 << 16, size=draw(st.integers(1, 5)), dtype=np.uint16)
        return vals[rng.integers(0, vals.size, size=n)]
    out = rng.integers(0, 1 << 16, size=n, dtype=np.uint16)    # NaN, Inf, zeros, denormals sprinkled in
    idx = rng.integers(0, n, size=64)
    out[idx] = rng.choice(np.array([0x7F80, 0xFF80, 0x7FC0, 0x0000, 0x8000, 0x0001, 0x807F], dtype=np.uint16), size=64)
    return out


@settings(max_examples=40, deadline=None, derandomize=True)
@given(tiles())
def test_any_tile_round_trips_and_never_grows(bits):
    x = _tile(bits)
    packed = K.reference_compress_tile(x)
    n = bits.size
    assert packed.numel() % 16 == 0 and packed.numel() <= 16 + 2 * n
    mode = int(packed[0])
    assert mode in (0, 1, 2)
    assert int.from_bytes(bytes(packed[4:8].numpy().tobytes()), "little") == packed.numel()
    back = K.reference_decompress_tile(packed)
    assert torch.equal(back.view(torch.int16), x.view(torch.int16))
    if mode:
        # the chosen shape is not longer than the other one for the sampled histogram (ties go to shape 1)
        C = n // K.CHUNK_VALS
        e = ((bits.astype(np.int64) >> 7) & 0xFF).reshape(K.CHUNK_VALS // 2, C, 2)
        hist = np.bincount(e[::K.SAMPLE_STRIDE].reshape(-1), minlength=256)
        order = sorted((b for b in range(256) if hist[b] > 0), key=lambda b: (-int(hist[b]), b))
        rank = {s: r for r, s in enumerate(order[:K.RANKS])}
        cost = {m: sum(int(hist[b]) * K._code_of(rank.get(b, K.RANKS), b, m)[1] for b in order) for m in (1, 2)}
        assert mode == (2 if cost[2] < cost[1] else 1)
        assert list(packed[16:16 + min(len(order), K.RANKS)].numpy()) == order[:K.RANKS]


@settings(max_examples=200, deadline=None, derandomize=True)
@given(st.lists(st.tuples(st.integers(0, K.RANKS), st.integers(0, 255), st.sampled_from([1, 2])), min_size=1, max_size=40))
def test_codes_are_prefix_free_and_self_delimiting(seq):
    """A stream of codes of either shape parses back to the same (rank or literal exponent) sequence."""
    for mode in (1, 2):
        acc, nb, want = 0, 0, []
        for rank, ex, _ in seq:
            code, ln = K._code_of(rank, ex, mode)
            assert 0 <= code < (1 << ln)
            acc |= code << nb
            nb += ln
            want.append(("lit", ex) if rank >= K.RANKS else ("rank", rank))
        got = []
        for _ in seq:
            if mode == 2:
                q = 0
                while (acc >> q) & 1 and q < K.FLAT_ESCAPE_ONES:
                    q += 1
                if q >= K.FLAT_ESCAPE_ONES:
                    got.append(("lit", (acc >> K.FLAT_ESCAPE_ONES) & 0xFF)); acc >>= K.FLAT_ESCAPE_ONES + 8
                else:
                    got.append(("rank", (q << 2) | ((acc >> (q + 1)) & 3))); acc >>= q + 3
            else:
                c = acc & 3
                if c != 3:
                    got.append(("rank", c)); acc >>= 2
                else:
                    t, ones = acc >> 2, 0
                    while (t >> ones) & 1 and ones < K.ESCAPE_ONES:
                        ones += 1
                    if ones >= K.ESCAPE_ONES:
                        got.append(("lit", (t >> K.ESCAPE_ONES) & 0xFF)); acc >>= 2 + K.ESCAPE_ONES + 8
                    else:
                        got.append(("rank", K.SHORT_RANKS + ones)); acc >>= ones + 3
        assert got == want and acc == 0
