"""Loading onto the device: through the two pinned staging buffers, experts stored one by one."""
import pytest
import torch

import helpers
import test_weights

pytestmark = pytest.mark.gpu


def test_upload_through_staging_buffers_and_one_by_one_experts(tmp_path):
    from quench6k_b200.engine import ModelRunner, StepEntry
    from quench6k_b200.models.flint import gguf_alias
    from quench6k_b200.weights import load_folder, write_safetensors
    from quench6k_b200.weights.loader import Uploader
    cfg, weights = helpers.make_model_folder(str(tmp_path), "B", seed=9)
    decl = test_weights._decl("B")
    # pieces far smaller than the tensors: every tensor crosses both buffers many times
    get = load_folder(str(tmp_path), decl, gguf_alias, device="cuda:0")
    get.uploader.piece = 1000
    get.uploader.buffers = [torch.empty(1000, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
    for spec in decl:
        t = get(spec.name)
        assert t.is_cuda and torch.equal(t.cpu(), weights[spec.name]), spec.name
    get.uploader.finish()
    toks = helpers.random_tokens(40, cfg["vocab_size"], 1)
    runner = ModelRunner.from_folder(str(tmp_path), dtype="float32", num_pages=8)
    runner.add_request("a")
    stacked = runner.step([StepEntry("a", toks, list(range(40)))]).cpu()
    write_safetensors(str(tmp_path / "model.safetensors"), test_weights._one_by_one(weights).items())
    runner = ModelRunner.from_folder(str(tmp_path), dtype="float32", num_pages=8)
    runner.add_request("a")
    assert torch.equal(runner.step([StepEntry("a", toks, list(range(40)))]).cpu(), stacked)
    helpers.assert_matches_plain(cfg, weights, toks, stacked, "float32", "experts stored one by one")


def test_device_generator_equals_the_host_and_numpy_twins_bit_for_bit():
    """The fill kernel, the C++ host generator and the NumPy twin: the same bits, in float32 and
    in bfloat16, from any offset; and a model made on the device equals the one made on the host."""
    import numpy as np
    import numpy_fill
    from quench6k_b200.weights.random_init import fill_normal, make_tensor
    for seed, name, start, count in ((0, "a", 0, 100003), (7, "model.layers.3.mlp.experts.gate_proj.weight", 123456789012, 4097)):
        for dtype in (torch.float32, torch.bfloat16):
            dev = fill_normal(torch.empty(count, dtype=dtype, device="cuda"), seed, name, start, 0.02, 1.0).cpu()
            host = fill_normal(torch.empty(count, dtype=dtype), seed, name, start, 0.02, 1.0)
            assert torch.equal(dev, host)
            twin = torch.from_numpy(numpy_fill.element_values(seed, name, start, count, 0.02, 1.0)).to(dtype)
            assert torch.equal(dev, twin)
    for spec in test_weights._decl("B"):
        assert torch.equal(make_tensor(spec, 3, 0.02, device="cuda").cpu(), make_tensor(spec, 3, 0.02)), spec.name
