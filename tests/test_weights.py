import os

import pytest
import torch

import helpers
import tiny_configs
from quench6k_b200.config import FlintConfig
from quench6k_b200.models.decoder import DecoderModel
from quench6k_b200.models.flint import build_spec
from quench6k_b200.spec import TensorSpec
from quench6k_b200.weights import (SafetensorsError, WeightError, index_folder, load_folder, make_tensor,
                                   standard_normal, write_safetensors)


def _decl(name="A"):
    return DecoderModel(build_spec(FlintConfig.from_dict(tiny_configs.get(name)))).tensors()


def test_random_folder_loads_back(tmp_path):
    cfg_d, weights = helpers.make_model_folder(str(tmp_path), "B", seed=3)
    decl = _decl("B")
    get = load_folder(str(tmp_path), decl)
    for spec in decl:
        t = get(spec.name)
        assert tuple(t.shape) == tuple(spec.shape)
        assert t.dtype == (torch.float32 if spec.role == "f32" else torch.bfloat16)
    assert os.path.exists(tmp_path / "config.json") and os.path.exists(tmp_path / "model.safetensors")


def test_seed_and_name_decide_the_values():
    s = TensorSpec("x.weight", (7, 5))
    a, b = make_tensor(s, 1, 0.02), make_tensor(s, 1, 0.02)
    assert torch.equal(a, b)
    assert not torch.equal(a, make_tensor(s, 2, 0.02))
    assert not torch.equal(a, make_tensor(TensorSpec("y.weight", (7, 5)), 1, 0.02))
    z = standard_normal(5, "n", 0, 200000, "cpu")
    assert abs(z.mean().item()) < 0.01 and abs(z.std().item() - 1.0) < 0.01
    # pieces of a tensor equal the whole
    assert torch.equal(standard_normal(5, "n", 1000, 50, "cpu"), z[1000:1050])
    ones = make_tensor(TensorSpec("n.weight", (9,), "f32", ("ones",)), 0, 0.02)
    assert ones.dtype == torch.float32 and torch.all(ones == 1)


def test_host_generator_equals_its_numpy_twin_bit_for_bit():
    """The C++ host generator against the NumPy twin under tests/: the same float32 bits, also
    through the scale, the mean and the rounding to bfloat16; and the values are what Box-Muller
    of the same uniforms gives in library arithmetic, to rounding."""
    import math
    import numpy as np
    import numpy_fill
    from quench6k_b200.weights.random_init import fill_normal, stream_key
    for seed, name, start, count in ((0, "a", 0, 5000), (7, "model.layers.3.mlp.experts.gate_proj.weight", 123456789012, 4097), (2**40 + 3, "x", 1 << 33, 1000)):
        assert stream_key(seed, name) == numpy_fill.stream_key(seed, name)
        z = standard_normal(seed, name, start, count, "cpu").numpy()
        twin = numpy_fill.standard_normal(seed, name, start, count)
        assert np.array_equal(z.view(np.uint32), twin.view(np.uint32))
        out = fill_normal(torch.empty(count, dtype=torch.float32), seed, name, start, 0.02, 1.0).numpy()
        assert np.array_equal(out.view(np.uint32), numpy_fill.element_values(seed, name, start, count, 0.02, 1.0).view(np.uint32))
        bf = fill_normal(torch.empty(count, dtype=torch.bfloat16), seed, name, start, 0.02, 0.0)
        assert torch.equal(bf, torch.from_numpy(numpy_fill.element_values(seed, name, start, count, 0.02, 0.0)).to(torch.bfloat16))
    # against the textbook formula with the library's log and cos
    key = np.uint64(numpy_fill.stream_key(5, "t"))
    with np.errstate(over="ignore"):
        j = np.arange(2000, dtype=np.uint64)
        a, b = numpy_fill._mix(j * np.uint64(2) + key), numpy_fill._mix(j * np.uint64(2) + np.uint64(1) + key)
    u1 = ((a >> np.uint64(11)).astype(np.float64) + 1.0) / 2.0**53
    u2 = (b >> np.uint64(11)).astype(np.float64) / 2.0**53
    want = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * math.pi * u2)
    got = standard_normal(5, "t", 0, 2000, "cpu").numpy().astype(np.float64)
    assert np.abs(got - want).max() <= 1e-6


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    cfg_d, weights = helpers.make_model_folder(str(tmp_path), "A", seed=0)
    bad = dict(weights)
    del bad["model.norm.weight"]
    del bad["model.layers.1.self_attn.o_proj.weight"]
    bad["model.layers.0.extra.bias"] = torch.zeros(3)
    bad["lm_head.weight"] = torch.zeros(10, 64, dtype=torch.bfloat16)
    bad["model.layers.0.mlp.gate.weight"] = torch.zeros(8, 64, dtype=torch.int32)
    write_safetensors(str(tmp_path / "model.safetensors"), bad.items())
    with pytest.raises(WeightError) as e:
        load_folder(str(tmp_path), _decl("A"))
    msg = str(e.value)
    assert "model.norm.weight" in msg and "model.layers.1.self_attn.o_proj.weight" in msg
    assert "model.layers.0.extra.bias" in msg
    assert "lm_head.weight: shape [10, 64], expected [256, 64]" in msg
    assert "model.layers.0.mlp.gate.weight: dtype" in msg
    assert e.value.missing == ["model.layers.1.self_attn.o_proj.weight", "model.norm.weight"]
    assert e.value.unexpected == ["model.layers.0.extra.bias"]
    assert len(e.value.wrong) == 2


def test_stored_dtypes_are_kept(tmp_path):
    write_safetensors(str(tmp_path / "model.safetensors"), [
        ("a", torch.randn(3, 4).to(torch.bfloat16)), ("b", torch.randn(5)), ("c", torch.arange(6, dtype=torch.int64)),
        ("d", torch.randn(2, 2).to(torch.float16))])
    decl = [TensorSpec("a", (3, 4)), TensorSpec("b", (5,), "f32"), TensorSpec("c", (6,), "i32"), TensorSpec("d", (2, 2))]
    get = load_folder(str(tmp_path), decl)
    assert get("a").dtype == torch.bfloat16 and get("b").dtype == torch.float32
    assert get("c").dtype == torch.int32 and get("c").tolist() == list(range(6))
    assert get("d").dtype == torch.bfloat16


def test_broken_files(tmp_path):
    with pytest.raises(SafetensorsError, match="no .safetensors"):
        index_folder(str(tmp_path))
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x10\x00\x00")
    with pytest.raises(SafetensorsError, match="shorter"):
        index_folder(str(tmp_path))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        index_folder(str(tmp_path))
    write_safetensors(str(p), [("a", torch.zeros(4))])
    write_safetensors(str(tmp_path / "other.safetensors"), [("a", torch.zeros(4))])
    with pytest.raises(SafetensorsError, match="duplicate tensor a"):
        index_folder(str(tmp_path))


def test_the_reference_names_are_accepted(tmp_path):
    """A checkpoint that names its tensors as the reference's GGUF does (blk.N.attn_q.weight, ...,
    expert tensors stacked as [E*I, D]) loads through the architecture's alias table; a tensor
    given under both names, or an aliased tensor of the wrong size, is reported."""
    from quench6k_b200.models.flint import gguf_alias
    src = tmp_path / "src"
    src.mkdir()
    _, weights = helpers.make_model_folder(str(src), "B", seed=4)
    decl = _decl("B")
    back = {}
    for n in weights:
        for cand in ["token_embd.weight", "output_norm.weight", "output.weight"] + [
                f"blk.{i}.{leaf}" for i in range(3) for leaf in (
                    "attn_norm.weight", "ffn_norm.weight", "attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight",
                    "attn_q_norm.weight", "attn_k_norm.weight", "attn_sinks.weight", "ffn_gate_inp.weight", "ffn_gate_exps.weight",
                    "ffn_up_exps.weight", "ffn_down_exps.weight", "ffn_gate_shexp.weight", "ffn_up_shexp.weight", "ffn_down_shexp.weight",
                    "ffn_gate.weight", "ffn_up.weight", "ffn_down.weight")]:
            if gguf_alias(cand) == n:
                back[n] = cand
    assert set(back) == set(weights)                      # every declared tensor has a name in the other scheme
    assert gguf_alias("blk.1.something_else") is None and gguf_alias("model.norm.weight") is None
    flat = lambda n, t: t.reshape(-1, t.shape[-1]) if "_exps" in back[n] else t
    other = tmp_path / "other"
    other.mkdir()
    write_safetensors(str(other / "model.safetensors"), [(back[n], flat(n, t)) for n, t in weights.items()])
    get = load_folder(str(other), decl, gguf_alias)
    for spec in decl:
        assert torch.equal(get(spec.name), weights[spec.name])
    with pytest.raises(WeightError, match="unexpected"):  # without the table the names mean nothing
        load_folder(str(other), decl)
    twice = tmp_path / "twice"
    twice.mkdir()
    write_safetensors(str(twice / "model.safetensors"), [(back[n], flat(n, t)) for n, t in weights.items()] +
                      [("model.norm.weight", weights["model.norm.weight"])])
    with pytest.raises(WeightError, match="stored twice"):
        load_folder(str(twice), decl, gguf_alias)
    wrong = tmp_path / "wrong"
    wrong.mkdir()
    write_safetensors(str(wrong / "model.safetensors"), [(back[n], flat(n, t)[:-1] if "_exps" in back[n] else t) for n, t in weights.items()])
    with pytest.raises(WeightError, match="wrong shape"):
        load_folder(str(wrong), decl, gguf_alias)


def test_both_readers_agree(tmp_path):
    """The C++ reader of safetensors files and its Python twin: the same entries and bytes for a
    file with metadata, escaped names, empty and scalar tensors; the same refusals for broken files."""
    import json
    import struct
    from quench6k_b200.weights.safetensors_io import SafetensorsFile
    good = tmp_path / "good.safetensors"
    tensors = [("plain", torch.randn(3, 5)), ("half.bf16", torch.randn(7).to(torch.bfloat16)), ("ints", torch.arange(12, dtype=torch.int64).reshape(2, 3, 2)),
               ("empty", torch.zeros(0, 4)), ("scalar", torch.tensor(2.5)), ('odd "name"\\ü\n', torch.ones(2, dtype=torch.uint8))]
    write_safetensors(str(good), tensors)
    raw = good.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    header["__metadata__"] = {"format": "pt", "note": "a \"quoted\" word", "nested": "x"}
    header["plain"]["extra_key"] = [1, {"a": None}, True, 1.5e3]
    blob = json.dumps(header, indent=1, ensure_ascii=True).encode()
    good.write_bytes(struct.pack("<Q", len(blob)) + blob + raw[8 + n:])
    a, b = SafetensorsFile(str(good), native=True), SafetensorsFile(str(good), native=False)
    assert a.entries == b.entries and set(a.entries) == {t[0] for t in tensors}
    for name, t in tensors:
        assert torch.equal(a.read(name), t) and torch.equal(b.read(name), t)

    def broken(data, match):
        p = tmp_path / "bad.safetensors"
        p.write_bytes(data)
        for native in (True, False):
            with pytest.raises(SafetensorsError, match=match):
                SafetensorsFile(str(p), native=native)

    def with_header(h, payload=b""):
        text = (h if isinstance(h, bytes) else json.dumps(h).encode())
        return struct.pack("<Q", len(text)) + text + payload

    broken(b"\x01\x02", "shorter than a safetensors header")
    broken(struct.pack("<Q", 100) + b"{}", "header length 100 exceeds the file")
    broken(with_header(b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]'), "header is not JSON")
    broken(with_header(b'[1, 2]'), "header is not JSON")
    broken(with_header({"a": {"dtype": "F8_E4M3", "shape": [1], "data_offsets": [0, 1]}}, b"\0"), "tensor a has unsupported dtype F8_E4M3")
    broken(with_header({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 8), "tensor a has byte range 0..4 for shape \\(2,\\) F32")
    broken(with_header({"a": {"dtype": "F32", "shape": [2, 1], "data_offsets": [0, 8]}}, b"\0" * 4), "tensor a has byte range 0..8 for shape \\(2, 1\\) F32 in a file of")
    broken(with_header({"a": {"dtype": "F32", "shape": [1]}}, b"\0" * 4), "tensor a lacks dtype, shape or data_offsets")


def test_header_reader_against_random_headers(tmp_path):
    """The C++ reader's own JSON reader against Python's on headers with random names (escapes,
    other scripts), random metadata values and unknown keys, written with random spacing."""
    import json
    import random
    import struct
    from quench6k_b200.weights.safetensors_io import SafetensorsFile
    rng = random.Random(17)
    alphabet = ['a', 'Z', '0', '.', '_', ' ', '"', '\\', '/', '\n', '\t', 'é', 'ß', '中', ' ', '\x7f', '{', ']', ':', ',']
    widths = {"F32": 4, "BF16": 2, "I64": 8, "U8": 1}

    def value(depth=0):
        kind = rng.randrange(7 if depth < 3 else 5)
        if kind == 0:
            return "".join(rng.choice(alphabet) for _ in range(rng.randrange(6)))
        if kind == 1:
            return rng.choice([0, -3, 17, 2.5, -1e-3, 6.02e23])
        if kind == 2:
            return rng.choice([True, False, None])
        if kind in (3, 4):
            return rng.randrange(1000)
        if kind == 5:
            return [value(depth + 1) for _ in range(rng.randrange(4))]
        return {str(i) + rng.choice(alphabet): value(depth + 1) for i in range(rng.randrange(4))}

    for case in range(40):
        header, at = {}, 0
        for t in range(rng.randrange(1, 7)):
            name = "".join(rng.choice(alphabet) for _ in range(rng.randrange(1, 12))) + str(t)
            dtype = rng.choice(list(widths))
            shape = [rng.randrange(0, 4) for _ in range(rng.randrange(0, 4))]
            n = widths[dtype]
            for d in shape:
                n *= d
            header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [at, at + n]}
            if rng.random() < 0.3:
                header[name]["note"] = value()
            at += n
        if rng.random() < 0.7:
            header["__metadata__"] = {"k" + str(i): value() for i in range(rng.randrange(4))}
        items = list(header.items())
        rng.shuffle(items)
        text = json.dumps(dict(items), ensure_ascii=rng.random() < 0.5, indent=rng.choice([None, 0, 3]),
                          separators=rng.choice([(",", ":"), (", ", ": "), (" ,\t", " :\n")])).encode()
        p = tmp_path / f"h{case}.safetensors"
        payload = bytes(rng.randrange(256) for _ in range(at))
        p.write_bytes(struct.pack("<Q", len(text)) + text + payload)
        a, b = SafetensorsFile(str(p), native=True), SafetensorsFile(str(p), native=False)
        assert a.entries == b.entries and len(a.entries) == len(header) - ("__metadata__" in header), case
        for name in a.entries:
            assert torch.equal(a.read(name).reshape(-1).view(torch.uint8), b.read(name).reshape(-1).view(torch.uint8))


def _one_by_one(weights):
    """The same checkpoint with every routed expert stored as a tensor of its own."""
    out = {}
    for n, t in weights.items():
        if ".mlp.experts." in n:
            stem, leaf = n.rsplit(".experts.", 1)
            for e in range(t.shape[0]):
                out[f"{stem}.experts.{e}.{leaf}"] = t[e].clone()
        else:
            out[n] = t
    return out


def test_experts_stored_one_by_one_are_stacked(tmp_path):
    """`mlp.experts.{e}.{gate,up,down}_proj.weight` are read into the stacked [E, ...] tensors the
    model declares; a missing expert, one too many and a wrong shape are all named in one error."""
    from quench6k_b200.models.flint import gguf_alias
    cfg_d, weights = helpers.make_model_folder(str(tmp_path), "A", seed=4)
    split = _one_by_one(weights)
    assert len(split) == len(weights) + 2 * 3 * (8 - 1)
    write_safetensors(str(tmp_path / "model.safetensors"), split.items())
    get = load_folder(str(tmp_path), _decl("A"), gguf_alias)
    for n, t in weights.items():
        assert torch.equal(get(n), t), n
    with pytest.raises(WeightError):                          # without the table of other names: 48 unexpected, 6 missing
        load_folder(str(tmp_path), _decl("A"))
    bad = dict(split)
    del bad["model.layers.1.mlp.experts.5.up_proj.weight"]
    bad["model.layers.0.mlp.experts.8.gate_proj.weight"] = torch.zeros(32, 64, dtype=torch.bfloat16)
    bad["model.layers.0.mlp.experts.2.down_proj.weight"] = torch.zeros(64, 31, dtype=torch.bfloat16)
    write_safetensors(str(tmp_path / "model.safetensors"), bad.items())
    with pytest.raises(WeightError) as e:
        load_folder(str(tmp_path), _decl("A"), gguf_alias)
    msg = str(e.value)
    assert "model.layers.1.mlp.experts.up_proj.weight[5]" in msg and "missing" in msg
    assert "model.layers.0.mlp.experts.8.gate_proj.weight" in msg and "unexpected" in msg
    assert "model.layers.0.mlp.experts.2.down_proj.weight: shape [64, 31], expected [64, 32]" in msg


def test_pieces_of_a_tensor_can_be_read(tmp_path):
    """What the upload through staging buffers reads: byte ranges of a tensor, by both readers."""
    t = torch.arange(1000, dtype=torch.float32).reshape(10, 100)
    write_safetensors(str(tmp_path / "x.safetensors"), [("pad", torch.zeros(3, dtype=torch.bfloat16)), ("t", t)])
    from quench6k_b200.weights import SafetensorsFile
    raw = t.view(-1).view(torch.uint8)
    for native in (True, False):
        sf = SafetensorsFile(str(tmp_path / "x.safetensors"), native=native)
        for off, n in ((0, 4000), (4, 8), (3996, 4), (1234, 1001), (50, 0)):
            out = torch.full((n,), 255, dtype=torch.uint8)
            sf.read_range("t", off, out)
            assert torch.equal(out, raw[off:off + n])
        with pytest.raises(SafetensorsError):
            sf.read_range("t", 3999, torch.zeros(2, dtype=torch.uint8))
