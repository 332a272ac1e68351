"""GPU tests of the module API: the reference's own inference tests, re-expressed against mlkit_b200.

They follow tests/inference/test_packed_linear.py, tests/checkpoints/test_checkpoints.py and
tests/conversion/test_head_quantization.py of the reference: packed output against the converted
(dense-reconstruction) model, every row count, every code width, offsets, layouts that split a word,
copies and casts, checkpoint round trips, packed embeddings and the online rotation hook.
"""

import copy

import numpy as np
import pytest
import torch
from torch import nn

import mlkit_b200 as mk
from mlkit_b200 import kernels
from oracle import matvec, transforms as oracle_transforms

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def seeded():
    torch.manual_seed(0)
    with torch.device("cuda"):
        yield


FORMATS = {"int4": mk.int(4, group=32), "nf4": mk.nf4(group=32)}


@pytest.mark.parametrize("name", FORMATS)
@pytest.mark.parametrize("batch", [1, 3, 7])
def test_packed_linear_matches_dense(name, batch):
    module = nn.Sequential(nn.Linear(130, 71, dtype=torch.float16))
    converted = mk.quantize(module, FORMATS[name], calib=None)
    packed = mk.optimize(converted, backend="packed")
    inputs = torch.randn(batch, 130, dtype=torch.float16)
    with torch.inference_mode():
        torch.testing.assert_close(packed(inputs), converted(inputs), rtol=0.002, atol=0.002)
    assert isinstance(packed.module[0], mk.PackedLinear)
    assert packed.module[0].packed.numel() == (130 * 71 + 1) // 2
    assert packed.execution_backend == "packed:1"


def packed_and_reference(format, *, input_width=256, output_width=37, dtype=torch.float32):
    module = nn.Sequential(nn.Linear(input_width, output_width, dtype=dtype))
    converted = mk.quantize(module, format, calib=None)
    packed = mk.optimize(converted, backend="packed")
    assert isinstance(packed.module[0], mk.PackedLinear)
    return packed, converted


@pytest.mark.parametrize("rows", [1, 2, 5, 8, 9, 33])
def test_packed_linear_handles_every_row_count(rows):
    packed, converted = packed_and_reference(mk.int(4, group=64))
    inputs = torch.randn(rows, 256)
    with torch.inference_mode():
        torch.testing.assert_close(packed(inputs), converted(inputs), rtol=1e-4, atol=1e-5)
        nested = inputs.reshape(1, rows, 256)
        torch.testing.assert_close(packed(nested), converted(nested), rtol=1e-4, atol=1e-5)


def test_packed_linear_applies_asymmetric_offsets():
    packed, converted = packed_and_reference(mk.int(4, group=64, asym=True))
    assert packed.module[0].zeros is not None
    for rows in (1, 3, 20):
        inputs = torch.randn(rows, 256)
        with torch.inference_mode():
            torch.testing.assert_close(packed(inputs), converted(inputs), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize(("input_width", "group"), [(255, 64), (256, 5), (250, 20)])
def test_layouts_that_split_a_packing_word_use_dense_reconstruction(input_width, group):
    packed, converted = packed_and_reference(mk.int(4, group=group), input_width=input_width)
    layer = packed.module[0]
    assert layer.layout is None and layer.maximum_fused_rows == 0
    inputs = torch.randn(2, input_width)
    with torch.inference_mode():
        torch.testing.assert_close(packed(inputs), converted(inputs), rtol=1e-4, atol=1e-5)
    assert torch.equal(layer.weight, converted.module[0].weight)


def test_packed_weight_reconstruction_is_bit_exact():
    for format in (mk.int(4, group=64), mk.nf4(group=32), mk.int(4, group=64, asym=True)):
        for dtype in (torch.float32, torch.float16):
            packed, converted = packed_and_reference(format, dtype=dtype)
            assert torch.equal(packed.module[0].weight, converted.module[0].weight)


def test_packed_linear_can_be_copied_and_cast_after_launching():
    packed, converted = packed_and_reference(mk.int(4, group=64), dtype=torch.float16)
    inputs = torch.randn(1, 256, dtype=torch.float16)
    with torch.inference_mode():
        expected = packed(inputs)
        duplicate = copy.deepcopy(packed)
        torch.testing.assert_close(duplicate(inputs), expected, rtol=0, atol=0)
        single = duplicate.module[0].float()
        result = single(inputs.float())
        torch.testing.assert_close(result, expected.float(), rtol=2e-3, atol=2e-3)
        assert result.dtype == torch.float32
        converted.module[0].weight.zero_()
        torch.testing.assert_close(packed(inputs), expected, rtol=0, atol=0)   # owns its storage
    assert packed.storage_bytes < converted.storage_bytes


WIDTH_FORMATS = {
    "int2": mk.int(2, group=64), "int3": mk.int(3, group=64), "int5": mk.int(5, group=64),
    "int6": mk.int(6, group=32), "int7": mk.int(7, group=64), "int8": mk.int(8, group=128),
    "int3-asymmetric": mk.int(3, group=64, asym=True), "e4m3": mk.scaled(mk.grid.fp("e4m3"), group=64),
    "codebook3": mk.scaled(mk.grid.values(torch.linspace(-1, 1, 7).pow(3), bits=3), group=32),
}


@pytest.mark.parametrize("name", WIDTH_FORMATS)
@pytest.mark.parametrize("rows", [1, 3, 20])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_packed_linear_executes_every_code_width(name, rows, dtype):
    packed, converted = packed_and_reference(WIDTH_FORMATS[name], dtype=dtype)
    layer = packed.module[0]
    bits = converted.quantized["0"].metadata["code_bits"]
    assert layer.layout is not None
    assert layer.packed.numel() == 37 * 256 * bits // 8
    inputs = torch.randn(rows, 256, dtype=dtype)
    with torch.inference_mode():
        tolerance = 1e-4 if dtype == torch.float32 else 2e-3
        torch.testing.assert_close(packed(inputs), converted(inputs), rtol=tolerance, atol=tolerance)
    assert torch.equal(layer.weight, converted.module[0].weight)


def test_three_bit_rows_that_split_a_word_use_dense_reconstruction():
    packed, converted = packed_and_reference(mk.int(3, group=50), input_width=250)
    assert packed.module[0].layout is None
    inputs = torch.randn(2, 250)
    with torch.inference_mode():
        torch.testing.assert_close(packed(inputs), converted(inputs), rtol=1e-4, atol=1e-5)


def test_wide_codes_remain_dense():
    converted = mk.quantize(nn.Sequential(nn.Linear(64, 16)), mk.int(12, group=32), calib=None)
    packed = mk.optimize(converted, backend="packed")
    assert isinstance(packed.module[0], nn.Linear)
    assert packed.execution_backend == "packed:0"


def test_error_behaviour_of_the_boundary():
    packed, _ = packed_and_reference(mk.int(4, group=64))
    layer = packed.module[0]
    with pytest.raises(ValueError, match="width"):
        layer(torch.randn(2, 255))
    with pytest.raises(ValueError, match="CUDA inputs"):
        layer(torch.randn(2, 256, device="cpu"))
    with pytest.raises(RuntimeError, match="autograd"):
        layer(torch.randn(2, 256, requires_grad=True))
    with pytest.raises(ValueError, match="QModel"):
        mk.optimize(nn.Linear(8, 8), backend="packed")
    bad = mk.Q(torch.zeros(37, 256))
    with pytest.raises(ValueError, match="scalar-grid codec"):
        mk.PackedLinear(nn.Linear(256, 37), bad)


def test_checkpoint_round_trip_preserves_outputs(tmp_path):
    module = nn.Sequential(nn.Linear(128, 48, bias=True, dtype=torch.float16), nn.ReLU(),
                           nn.Linear(48, 16, bias=False, dtype=torch.float16))
    converted = mk.quantize(module, mk.nf4(group=16), calib=None)
    packed = mk.optimize(converted)
    inputs = torch.randn(4, 128, dtype=torch.float16)
    with torch.inference_mode():
        expected = packed(inputs)
    packed.save(tmp_path / "packed")
    with pytest.raises(FileExistsError):
        packed.save(tmp_path / "packed")
    packed.save(tmp_path / "packed", overwrite=True)
    factory = lambda: nn.Sequential(nn.Linear(128, 48, bias=True), nn.ReLU(), nn.Linear(48, 16, bias=False))
    restored = mk.load(tmp_path / "packed", model=factory)
    assert set(restored.quantized) == {"0", "2"}
    with torch.inference_mode():
        torch.testing.assert_close(restored(inputs), converted(inputs), rtol=0, atol=0)
        repacked = mk.optimize(restored)
        assert repacked.execution_backend == "packed:2"
        torch.testing.assert_close(repacked(inputs), expected, rtol=0, atol=0)
    import json

    manifest = json.loads((tmp_path / "packed" / "mlkit.json").read_text())
    assert manifest["format_version"] == 1 and manifest["layers"]["0"]["codec"] == "scaled"
    assert manifest["layers"]["2"]["params"]["values"]["tensor"] == "0.params.values"   # stored once
    from safetensors.torch import load_file

    stored = load_file(str(tmp_path / "packed" / "weights.safetensors"))
    assert stored["0.codes"].numel() == 128 * 48 // 2 and stored["0.params.scales"].dtype == torch.float16
    assert manifest["tensor_bytes"] == sum(v.numel() * v.element_size() for v in stored.values())


class TiedModel(nn.Module):
    def __init__(self):
        super().__init__()
        self.embedding = nn.Embedding(40, 64)
        self.head = nn.Linear(64, 40, bias=False)
        self.head.weight = self.embedding.weight

    def forward(self, ids):
        return self.head(self.embedding(ids))


def test_packed_embedding_reads_rows_of_the_packed_head():
    module = TiedModel().half()
    converted = mk.quantize(module, mk.int(4, group=32), calib=None)
    converted.tied_weights = {"embedding.weight": "head"}
    packed = mk.optimize(converted, backend="packed")
    assert isinstance(packed.module.embedding, mk.PackedEmbedding)
    ids = torch.tensor([[0, 5, 39], [7, 7, 1]])
    with torch.inference_mode():
        rows = packed.module.embedding(ids)
        assert torch.equal(rows, converted.module.embedding(ids))
        torch.testing.assert_close(packed(ids), converted(ids), rtol=2e-3, atol=2e-3)
    assert torch.equal(packed.module.embedding.weight, converted.module.head.weight)


@pytest.mark.parametrize("width", [4096, 14336, 896])
def test_online_rotation_hook_preserves_the_layer_function(width, tmp_path):
    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.down_proj = nn.Linear(width, 64, bias=False, dtype=torch.float16)

        def forward(self, x):
            return self.down_proj(x)

    block = Block()
    with torch.no_grad():
        block.down_proj.weight.mul_(0.5)
    inputs = torch.randn(8, width, dtype=torch.float16)
    outlier_channels = torch.randperm(width)[: width // 100]
    inputs[:, outlier_channels] *= 50
    with torch.inference_mode():
        plain = block(inputs).float()
    mk.rotate_inputs(block, seed=3)
    descriptor = block._mlkit_transforms[0]
    assert descriptor == {"kind": "rotation", "name": "down_proj", "seed": mk.layer_seed("down_proj", 3)}
    with torch.inference_mode():
        rotated_dense = block(inputs).float()
    assert matvec.relative_l2(rotated_dense.cpu().numpy(), plain.cpu().numpy()) < 5e-3
    converted = mk.quantize(block, mk.int(4, group=128), calib=None)
    packed = mk.optimize(converted, backend="packed")
    with torch.inference_mode():
        out = packed(inputs[:1]), packed(inputs)
        reference = converted(inputs)
    assert matvec.relative_l2(out[1].float().cpu().numpy(), reference.float().cpu().numpy()) < 2e-3
    assert matvec.relative_l2(out[0].float().cpu().numpy(), reference[:1].float().cpu().numpy()) < 2e-3
    # the hook equals the oracle's randomized transform with the same signs
    hook = next(iter(packed.module.down_proj._forward_pre_hooks.values()))
    signs = hook.signs_for(width, inputs.device).cpu().numpy()
    got = mk.rht(inputs, signs=hook.signs_for(width, inputs.device)).float().cpu().numpy()
    expected = oracle_transforms.randomized_transform(inputs.float().cpu().numpy(), signs, by_multiply=True)
    assert matvec.relative_l2(got, expected) < 2e-3
    # checkpoints keep the transform
    packed.save(tmp_path / "rotated")
    restored = mk.optimize(mk.load(tmp_path / "rotated", model=lambda: Block().float()))
    with torch.inference_mode():
        torch.testing.assert_close(restored(inputs), out[1], rtol=0, atol=0)


def test_transform_api_matches_oracle():
    values = torch.randn(12, 64)
    torch.testing.assert_close(mk.hadamard(mk.hadamard(values)), values, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(mk.rht(mk.rht(values, seed=4), seed=4, inverse=True), values, rtol=1e-5, atol=1e-5)
    for width in [12, 20, 28, 96, 896, 4864, 7]:
        x = torch.randn(3, width)
        y = mk.structured_transform(x)
        torch.testing.assert_close(mk.structured_transform(y, inverse=True), x, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(y.square().sum(1), x.square().sum(1), rtol=1e-5, atol=1e-5)
        expected = oracle_transforms.structured_transform(x.cpu().numpy(), by_multiply=True)
        assert matvec.relative_l2(y.cpu().numpy(), expected) < 1e-6


def test_compiled_module_traces_the_custom_op():
    packed, converted = packed_and_reference(mk.int(4, group=64), dtype=torch.float16)
    inputs = torch.randn(2, 256, dtype=torch.float16)
    with torch.inference_mode():
        eager = packed(inputs)
        compiled = torch.compile(packed.module, fullgraph=True)
        torch.testing.assert_close(compiled(inputs), eager, rtol=0, atol=0)


def test_benchmark_protocol():
    packed, _ = packed_and_reference(mk.int(4, group=64))
    inputs = torch.randn(1, 256)
    result = mk.benchmark_model(packed, inputs, warmup=1, repetitions=3)
    assert result.median_ms > 0 and result.repetitions == 3 and result.minimum_ms <= result.percentile_95_ms
    assert set(result.to_dict()) == {"median_ms", "minimum_ms", "percentile_95_ms", "repetitions", "device",
                                     "peak_memory_bytes"}


class LlamaishBlock(nn.Module):
    """The seven linears of a Llama block under the names the sibling grouping looks for."""

    def __init__(self, hidden=512, kv=128, mlp=1024):
        super().__init__()
        self.q_proj = nn.Linear(hidden, hidden, bias=False, dtype=torch.float16)
        self.k_proj = nn.Linear(hidden, kv, bias=False, dtype=torch.float16)
        self.v_proj = nn.Linear(hidden, kv, bias=False, dtype=torch.float16)
        self.o_proj = nn.Linear(hidden, hidden, bias=False, dtype=torch.float16)
        self.gate_proj = nn.Linear(hidden, mlp, bias=False, dtype=torch.float16)
        self.up_proj = nn.Linear(hidden, mlp, bias=False, dtype=torch.float16)
        self.down_proj = nn.Linear(mlp, hidden, bias=False, dtype=torch.float16)

    def forward(self, x):
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        attended = self.o_proj(q * torch.sigmoid(k.mean(-1, keepdim=True)) + v.mean(-1, keepdim=True))
        return self.down_proj(nn.functional.silu(self.gate_proj(attended)) * self.up_proj(attended))


@pytest.mark.parametrize("rows", [1, 8])
def test_sibling_projections_share_one_launch_bit_for_bit(rows):
    converted = mk.quantize(LlamaishBlock(), mk.int(4, group=128), calib=None)
    fused = mk.optimize(converted, backend="packed")
    separate = mk.optimize(converted, backend="packed", siblings=None)
    block = fused.module
    assert block.q_proj._siblings is block.k_proj._siblings is block.v_proj._siblings is not None
    assert block.gate_proj._siblings is block.up_proj._siblings is not None
    assert block.o_proj._siblings is None and separate.module.q_proj._siblings is None
    # the members' buffers are views of one allocation, so checkpoints and state dicts are unchanged
    assert block.k_proj.packed.data_ptr() == block.q_proj.packed.data_ptr() + block.q_proj.packed.numel()
    assert torch.equal(block.v_proj.packed, separate.module.v_proj.packed)
    x = torch.randn(rows, 512, dtype=torch.float16)
    with torch.inference_mode():
        for name in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj"):
            assert torch.equal(getattr(block, name)(x), getattr(separate.module, name)(x)), name
        assert torch.equal(fused(x), separate(x))
        torch.testing.assert_close(fused(x), converted(x), rtol=0.01, atol=0.01)
    # one launch serves each member once: a second call of the same member, a changed input and a new
    # tensor all start a new launch and see the new values
    y = torch.randn(rows, 512, dtype=torch.float16)
    first = block.q_proj(y).clone()
    assert torch.equal(block.q_proj(y), first)
    assert torch.equal(block.k_proj(y), separate.module.k_proj(y))
    y.mul_(2)
    assert torch.equal(block.v_proj(y), separate.module.v_proj(y))
    assert torch.equal(block.k_proj(y), separate.module.k_proj(y))
    # rows beyond the fused limit take the dense route per member, as before
    many = torch.randn(9, 512, dtype=torch.float16)
    torch.testing.assert_close(block.k_proj(many), separate.module.k_proj(many))
    # moving a member dissolves the group; every member then launches alone
    block.q_proj.half()
    assert block.k_proj._siblings is None
    assert torch.equal(block.k_proj(x), separate.module.k_proj(x))


# ---------------------------------------------------------------- a checkpoint written by the reference
GOLDEN_CHECKPOINTS = __import__("pathlib").Path(__file__).resolve().parent / "golden" / "ckpt"


class TiedLanguageModel(nn.Module):
    """The model of the reference's checkpoint test (tests/checkpoints/test_checkpoints.py:60-80)."""

    def __init__(self):
        super().__init__()
        self.embedding = nn.Embedding(32, 16)
        self.projections = nn.Sequential(nn.Linear(16, 16), nn.Linear(16, 16))
        self.lm_head = nn.Linear(16, 32, bias=False)
        self.lm_head.weight = self.embedding.weight

    def forward(self, tokens):
        return self.lm_head(self.projections(self.embedding(tokens)))


def _stored_tensors(directory):
    from safetensors import safe_open

    with safe_open(str(directory / "weights.safetensors"), "pt") as handle:
        return {key: handle.get_tensor(key) for key in handle.keys()}


def test_checkpoint_written_by_the_reference_loads_runs_and_saves_back(tmp_path):
    """``tests/golden/ckpt/tied`` was written by the reference's own ``save`` (see make_checkpoint.py
    beside it).  It must load unchanged, reproduce the reference's outputs, run packed, and a re-save
    must give the same manifest entries and the same tensors, key for key and byte for byte."""
    import json

    source = GOLDEN_CHECKPOINTS / "tied"
    stored = np.load(GOLDEN_CHECKPOINTS / "tied_io.npz")
    tokens, expected = torch.from_numpy(stored["tokens"]).cuda(), torch.from_numpy(stored["logits"]).cuda()
    restored = mk.load(source, model=TiedLanguageModel)
    assert restored.module.embedding.weight is restored.module.lm_head.weight
    with torch.inference_mode():
        torch.testing.assert_close(restored(tokens), expected, rtol=1e-5, atol=1e-6)
        packed = mk.optimize(restored)
        assert packed.execution_backend == "packed:2"
        assert matvec.relative_l2(packed(tokens).float().cpu().numpy(), stored["logits"]) < 2e-3
    restored.save(tmp_path / "again")
    first, second = json.loads((source / "mlkit.json").read_text()), json.loads((tmp_path / "again" / "mlkit.json").read_text())
    for key in ("format_version", "name", "architecture", "dtype", "layers", "logical_bpw", "model_bpw",
                "parameter_accounting", "transforms", "activations", "kv", "state_aliases", "tied_weights", "tensor_bytes"):
        assert first[key] == second[key], key
    before, after = _stored_tensors(source), _stored_tensors(tmp_path / "again")
    assert set(before) == set(after)
    for key, value in before.items():
        assert value.dtype == after[key].dtype and torch.equal(value, after[key]), key


def test_reference_checkpoint_with_a_rotation_installs_the_hook(tmp_path):
    """``tests/golden/ckpt/rotated``: the manifest carries the rotation descriptor the reference
    recorded; loading installs the input hook and a re-save keeps descriptor and tensors."""
    import json

    class Attention(nn.Module):
        def __init__(self):
            super().__init__()
            self.o_proj = nn.Linear(64, 24, bias=False)

        def forward(self, x):
            return self.o_proj(x)

    source = GOLDEN_CHECKPOINTS / "rotated"
    seed = json.loads((GOLDEN_CHECKPOINTS / "fixture.json").read_text())["rotated"]["seed"]
    restored = mk.load(source, model=Attention)
    assert len(restored.module.o_proj._forward_pre_hooks) == 1
    assert restored.module._mlkit_transforms == [{"kind": "rotation", "name": "o_proj", "seed": seed}]
    x = torch.randn(3, 64)
    packed = mk.optimize(restored)
    with torch.inference_mode():
        # the hook rotates with this device's sign vector, in the dense and in the packed model alike
        expected = torch.nn.functional.linear(mk.rht(x, seed=seed), restored.module.o_proj.weight)
        torch.testing.assert_close(restored(x), expected, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(packed(x), expected, rtol=2e-3, atol=2e-3)
    restored.save(tmp_path / "again")
    again = json.loads((tmp_path / "again" / "mlkit.json").read_text())
    assert again["transforms"] == json.loads((source / "mlkit.json").read_text())["transforms"]
    before, after = _stored_tensors(source), _stored_tensors(tmp_path / "again")
    assert set(before) == set(after) and all(torch.equal(before[key], after[key]) for key in before)


def test_captured_call_matches_eager_with_device_and_host_inputs():
    """``mk.capture``: one graph per input signature; host inputs (pinned or not) and host results are
    copy nodes of the graph.  Every replay equals the eager call bit for bit, also after the input's
    contents change and with sibling launches inside the captured module."""
    import torch.nn as nn

    class Pair(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj = nn.Linear(256, 384, bias=False)
            self.up_proj = nn.Linear(256, 384, bias=False)
            self.down_proj = nn.Linear(384, 256, bias=True)

        def forward(self, x):
            hidden = torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x)
            return self.down_proj(hidden), hidden

    torch.manual_seed(3)
    model = Pair().half().cuda()
    quantized = mk.quantize(model, mk.int(4, group=128))
    fast = mk.optimize(quantized, backend="packed")
    assert fast.module.gate_proj._siblings is not None
    call = mk.capture(fast.module)
    with torch.inference_mode():
        for rows in (1, 3):
            for trial in range(3):
                x = torch.randn(rows, 256, device="cuda").half()
                expected = [t.clone() for t in fast.module(x)]
                got = call(x)
                assert all(t.is_cuda for t in got)
                assert all(torch.equal(a, b) for a, b in zip(got, expected))
                pinned = x.cpu().pin_memory()
                for host in (x.cpu(), pinned):
                    got = call(host)
                    assert all(not t.is_cuda for t in got)
                    assert all(torch.equal(a, b.cpu()) for a, b in zip(got, expected))
                # a pinned input is read in place: new contents, same address, same graph
                pinned.copy_(-x.cpu())
                expected = [t.clone() for t in fast.module(-x)]
                got = call(pinned)
                assert all(torch.equal(a, b.cpu()) for a, b in zip(got, expected))
    assert len(call.entries) == 2 * (1 + 1 + 3)   # per row count: device, pageable host, one pinned tensor per trial
    lazy = mk.capture(fast.module, synchronize=False)
    host = torch.randn(2, 256, device="cpu").half().pin_memory()
    out = lazy(host)
    lazy.wait()
    with torch.inference_mode():
        assert torch.equal(out[0], fast.module(host.cuda())[0].cpu())


def test_device_encoder_stream_is_reused_only_while_codes_are_untouched():
    weight = torch.randn(48, 256, device="cuda")
    q = mk.int(4, group=128)(weight, mk.Ctx("layer", device="cuda"))
    assert q._stream is not None
    assert torch.equal(q.packed_stream(4), mk.pack(q.codes, 4))
    assert q.packed_stream(4) is q._stream[0]
    q.codes[0, 0] = (q.codes[0, 0] + 1) % 16          # in-place edit: the stream on record is stale
    assert q.packed_stream(4) is not q._stream[0]
    assert torch.equal(q.packed_stream(4), mk.pack(q.codes, 4))


def test_rotated_packed_linear_fuses_the_rotation_for_few_rows():
    """With at most M * K * 4 <= 16 KB of activations (where the fused launch is the faster one) the rotation
    hook hands its sign vector to the layer, which rotates while it loads (``mkb_gemv_hadamard``); the output
    equals the two launches bit for bit, and the hook still rotates by itself for more rows and when another
    hook follows it."""
    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.o_proj = nn.Linear(2048, 96, bias=True, dtype=torch.float16)

        def forward(self, x):
            return self.o_proj(x)

    torch.manual_seed(5)
    block = Block()
    mk.rotate_inputs(block, seed=11)
    packed = mk.optimize(mk.quantize(block, mk.int(4, group=128), calib=None), backend="packed")
    layer = packed.module.o_proj
    inputs = torch.randn(8, 2048, dtype=torch.float16)
    calls = []
    original = kernels.packed_matvec_rotated
    kernels.packed_matvec_rotated = lambda *a, **k: (calls.append(a[0].shape[0]), original(*a, **k))[1]
    try:
        with torch.inference_mode():
            fused = [packed(inputs[:rows]) for rows in (1, 2, 8)]
            layer._rotation_refused = True
            separate = [packed(inputs[:rows]) for rows in (1, 2, 8)]
            layer._rotation_refused = False
            layer.register_forward_pre_hook(lambda module, arguments: None)   # a later hook: the fusion stands down
            after = packed(inputs[:1])
    finally:
        kernels.packed_matvec_rotated = original
    assert calls == [1, 2]             # 2 x 2048 x 4 B = 16 KB is the limit; nothing fused after the later hook
    assert all(torch.equal(a, b) for a, b in zip(fused, separate))
    assert torch.equal(after, separate[0])


def test_captured_call_bounds_its_graphs_per_pinned_address():
    """A pinned input is read in place, so its address keys a graph of its own; a caller that brings a new pinned
    tensor every time must not grow one graph per call: past the bound such inputs are staged like pageable ones."""
    linear = torch.nn.Linear(256, 128, bias=False).half().cuda()
    call = mk.capture(linear)
    call.MAXIMUM_PINNED_CAPTURES = 4
    with torch.inference_mode():
        for trial in range(10):
            x = torch.randn(2, 256, device="cpu").half().pin_memory()
            assert torch.equal(call(x), linear(x.cuda()).cpu())
    assert len(call.entries) == 5          # four graphs keyed by address, then one staged graph for the shape
    again = torch.randn(2, 256, device="cpu").half().pin_memory()
    with torch.inference_mode():
        assert torch.equal(call(again), linear(again.cuda()).cpu()) and torch.equal(call(again), linear(again.cuda()).cpu())
    assert len(call.entries) == 5
