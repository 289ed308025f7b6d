"""Weights I/O on the device: a safetensors file with an MLX 4-bit checkpoint layout is validated, mapped and
imported as one read-only buffer; its tensors are views of that buffer that the operators read directly."""
import json
import struct

import numpy as np
import pytest

import forja_b200 as fb
from forja_b200 import weights as W
from forja_b200.backend import Op
from oracle import fjo
from tests.gpu_util import QUANT_TOL, assert_close, backend, down, down_raw, up

pytestmark = pytest.mark.gpu


def write_safetensors(path, tensors):
    """tensors: {name: (dtype name, numpy array)}; data laid out in insertion order."""
    header, blobs, cursor = {}, [], 0
    for name, (dtype, array) in tensors.items():
        raw = np.ascontiguousarray(array).tobytes()
        header[name] = {"dtype": dtype, "shape": list(array.shape), "data_offsets": [cursor, cursor + len(raw)]}
        blobs.append(raw)
        cursor += len(raw)
    text = json.dumps(header).encode()
    text += b" " * (-(len(text) + 8) % 8)
    path.write_bytes(struct.pack("<Q", len(text)) + text + b"".join(blobs))


def test_imported_mlx_4bit_checkpoint_feeds_quant_matmul_and_embed(tmp_path):
    rng = np.random.default_rng(3)
    be = backend()
    k, n, experts = 256, 96, 3
    packed = rng.integers(0, 2 ** 32, (n, k // 8), dtype=np.uint64).astype(np.uint32)
    scales = fjo.encode((rng.standard_normal((n, k // 64)) * 0.01).astype(np.float32), fb.BF16)
    biases = fjo.encode((rng.standard_normal((n, k // 64)) * 0.01).astype(np.float32), fb.BF16)
    table = fjo.encode(rng.standard_normal((50, 32)).astype(np.float32), fb.BF16)
    stack = rng.integers(0, 2 ** 32, (experts, n, k // 8), dtype=np.uint64).astype(np.uint32)
    stack_s = fjo.encode((rng.standard_normal((experts, n, k // 64)) * 0.01).astype(np.float32), fb.BF16)
    path = tmp_path / "model.safetensors"
    write_safetensors(path, {
        "model.norm.weight": ("BF16", table[0]),
        "model.layers.0.self_attn.q_proj.weight": ("U32", packed),
        "model.layers.0.self_attn.q_proj.scales": ("BF16", scales),
        "model.layers.0.self_attn.q_proj.biases": ("BF16", biases),
        "model.embed_tokens.weight": ("BF16", table),
        "model.layers.0.mlp.switch_mlp.gate_proj.weight": ("U32", stack),
        "model.layers.0.mlp.switch_mlp.gate_proj.scales": ("BF16", stack_s),
        "model.layers.0.mlp.switch_mlp.gate_proj.biases": ("BF16", stack_s),
    })
    source = W.Safetensors.open(path)
    used_before = be.memory_usage()[0]
    imported = source.import_into(be)
    assert be.memory_usage()[0] - used_before == source.file_len - source.data_start
    # plain tensors are byte-identical views
    embed = imported.tensor("model.embed_tokens.weight")
    assert embed.shape == (50, 32) and not embed.writable
    assert np.array_equal(down_raw(embed), table)
    # the quantised triple runs through Op::QuantMatmul as imported
    p, s, b = imported.quant("model.layers.0.self_attn.q_proj")
    assert p.shape == (n, k // 8) and s.shape == (n, k // 64)
    x, xh = up(rng.standard_normal((5, k)), fb.BF16)
    out = be.alloc(fb.BF16, (5, n))
    be.run(Op.QuantMatmul(4, 64), [x, p, s, b], [out])
    want = fjo.quant_matmul(xh, fb.BF16, packed, scales, biases, fb.BF16, 4, 64)
    assert_close(down(out), fjo.decode(want, fb.BF16), QUANT_TOL)
    ep, es, eb = imported.quant("model.layers.0.mlp.switch_mlp.gate_proj")
    assert ep.shape == (experts, n, k // 8) and es.shape == eb.shape == (experts, n, k // 64)
    # a read-only import cannot be an output
    with pytest.raises(fb.BackendError):
        be.run(Op.Copy(), [x], [imported.tensor("model.norm.weight")])
    # shape cross-checks of the triple
    with pytest.raises(fb.BackendError):
        imported.quant("model.layers.0.self_attn.q_proj", bits=8)
    with pytest.raises(fb.BackendError):
        imported.quant("model.layers.0.self_attn.k_proj")
    be.release(embed)
