"""Property tests (hypothesis): placements tile a tensor exactly, byte spans rebuild shards, float codecs and
tokenizers round-trip."""
import numpy as np
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st  # noqa: E402

from zml_b200 import Shape, floats  # noqa: E402
from zml_b200.sharding import TORUS, LogicalMesh, PhysicalMesh, Sharding, Strategy  # noqa: E402

MESHES = [(2,), (4,), (8,), (2, 2), (2, 4), (2, 2, 2)]
TAGS = ("link_x", "link_y", "link_z")


@st.composite
def sharded_case(draw):
    mesh = draw(st.sampled_from(MESHES))
    phys_tags = TAGS[:len(mesh)]
    rank = draw(st.integers(1, 3))
    # every logical axis is bound to a distinct non-empty subset of the mesh axes; tensor axes use distinct logical axes
    axes = list(phys_tags)
    draw(st.randoms(use_true_random=False)).shuffle(axes)
    n_logical = draw(st.integers(0, min(rank, len(axes))))
    bindings, used = {}, 0
    for i in range(n_logical):
        take = draw(st.integers(1, len(axes) - used - (n_logical - i - 1)))
        bindings[f"l{i}"] = axes[used:used + take]
        used += take
    sizes = dict(zip(phys_tags, mesh))
    dims, specs = [], {}
    which = draw(st.permutations(range(rank)))
    for ax in range(rank):
        mult = draw(st.integers(1, 3))
        if which.index(ax) < n_logical:
            name = f"l{which.index(ax)}"
            parts = int(np.prod([sizes[p] for p in bindings[name]]))
            dims.append(parts * mult)
            specs[ax] = name
        else:
            dims.append(mult + 1)
            specs[ax] = draw(st.sampled_from(["replicated", "unknown", "open"]))
    return mesh, phys_tags, bindings, tuple(dims), specs


@settings(max_examples=120, deadline=None, derandomize=True)
@given(sharded_case())
def test_placement_tiles_the_tensor_and_byte_spans_rebuild_every_shard(case):
    mesh, phys_tags, bindings, dims, specs = case
    phys = PhysicalMesh.grid(mesh, TORUS, phys_tags, target="tpu")
    bound = bindings or {"unused": [phys_tags[0]]}          # a binding no tensor axis names leaves everything replicated
    logical = LogicalMesh.mesh({k: "high_bandwidth" for k in bound})
    sharding = Sharding("s", phys, logical, Strategy.parse_bindings(bound))
    shape = Shape(dims, "i32").with_partitioning(specs)
    pl = sharding.placement(shape)
    full = np.arange(int(np.prod(dims)), dtype=np.int32).reshape(dims)
    cover = np.zeros(dims, dtype=np.int64)
    raw = full.tobytes()
    n_parts = 1
    for ax, s in specs.items():
        if s in bindings:
            n_parts *= int(np.prod([dict(zip(phys_tags, mesh))[p] for p in bindings[s]]))
    for dev in phys.devices:
        idx = pl.shard_index(dev)
        shard = full[idx]
        assert shard.shape == tuple(pl.shape.dims)
        cover[idx] += 1
        # the byte spans of the row-major global array, concatenated, are the shard in row-major order
        rebuilt = b"".join(raw[o:o + n] for o, n in pl.byte_spans(dev))
        assert rebuilt == np.ascontiguousarray(shard).tobytes()
    # every element is held by the same number of devices: devices / partitions
    assert (cover == len(phys.devices) // n_parts).all()
    # annotations agree with the placement on the tile counts
    attr = sharding.gspmd_sharding_attr(shape)
    if n_parts == 1:
        assert attr == "{replicated}"
    else:
        tiles = [int(t) for t in attr[attr.index("[") + 1:attr.index("]")].split(",")]
        assert int(np.prod(tiles)) == len(phys.devices) and tiles[:len(dims)] == [d // l for d, l in zip(dims, pl.shape.dims)]


@pytest.mark.parametrize("name", ["f8e4m3fn", "f8e4m3fnuz", "f8e5m2", "f8e5m2fnuz", "f8e4m3", "f8e3m4", "f8e4m3b11fnuz", "f4e2m1", "bf16"])
def test_every_code_of_a_float_format_round_trips(name):
    fmt = floats.FORMATS[name]
    codes = np.arange(1 << min(fmt.bits, 16), dtype=np.uint32 if fmt.bits > 8 else np.uint8)
    vals = fmt.to_f32(codes)
    back = fmt.from_f32(vals).astype(np.int64)
    ok = (back == codes.astype(np.int64)) | np.isnan(vals)            # NaNs come back as the canonical NaN
    if fmt.flavour == "fnuz":
        ok |= vals == 0                                               # one zero only
    assert ok.all(), (name, codes[~ok][:8], vals[~ok][:8])
    finite = vals[np.isfinite(vals)]
    assert finite.max() == fmt.max_finite and finite.min() == -fmt.max_finite


@settings(max_examples=200, deadline=None, derandomize=True)
@given(st.floats(allow_nan=False, allow_infinity=False, width=32), st.sampled_from(["f8e4m3fn", "f8e5m2", "bf16", "f4e2m1"]))
def test_float_encoding_is_the_nearest_code(x, name):
    fmt = floats.FORMATS[name]
    got = float(fmt.to_f32(fmt.from_f32(np.float32(x), saturate=True)))
    grid = fmt.to_f32(np.arange(1 << min(fmt.bits, 16)))
    grid = np.unique(grid[np.isfinite(grid)])
    xs = float(np.clip(np.float32(x), -fmt.max_finite, fmt.max_finite))
    best = float(np.min(np.abs(grid.astype(np.float64) - xs)))
    assert abs(got - xs) <= best * (1 + 1e-6) + 1e-45, (x, got, best)


@settings(max_examples=60, deadline=None, derandomize=True)
@given(st.text(alphabet=st.characters(blacklist_categories=("Cs",), blacklist_characters="\x00"), max_size=40))
def test_byte_level_bpe_round_trips_any_text(text):
    tok = _bpe()
    ids = tok.encode(text)
    assert tok.decode(ids) == text
    dec = tok.decoder()
    assert "".join(dec.next(i) for i in ids) + dec.finalize() == text


_BPE = None


def _bpe():
    global _BPE
    if _BPE is None:
        tokenizers = pytest.importorskip("tokenizers")
        from tokenizers import Tokenizer as HfTok, decoders, models, pre_tokenizers, trainers
        from zml_b200.tokenizer import Tokenizer
        t = HfTok(models.BPE())
        t.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
        t.decoder = decoders.ByteLevel()
        t.train_from_iterator(["hello world, the quick brown fox jumps over the lazy dog 0123456789"] * 20,
                              trainers.BpeTrainer(vocab_size=400, initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
        _BPE = Tokenizer.from_bytes(t.to_str().encode(), backend="homemade")
    return _BPE


@given(text=st.text(alphabet="ab c", max_size=40), stops=st.lists(st.text(alphabet="ab c", min_size=1, max_size=4), max_size=3),
       cuts=st.lists(st.integers(0, 40), max_size=8))
@settings(max_examples=300, deadline=None, derandomize=True)
def test_streamed_stop_filter_equals_cutting_the_whole_text(text, stops, cuts):
    """However the text is split into pieces, what the filter lets through adds up to the text cut at the first stop
    string, nothing is sent after a stop, and a stop is reported exactly when the text holds one."""
    from zml_b200.serving.server import StopFilter, _first_stop
    bounds = sorted({min(c, len(text)) for c in cuts} | {0, len(text)})
    pieces = [text[a:b] for a, b in zip(bounds, bounds[1:])] or [""]
    f = StopFilter(stops)
    sent, stopped = "", False
    for i, piece in enumerate(pieces):
        out, now = f.feed(piece, i == len(pieces) - 1)
        assert not (stopped and out)
        sent += out
        stopped = stopped or now
    cut = _first_stop(text, stops)
    assert sent == (text if cut < 0 else text[:cut]) and stopped == (cut >= 0)
