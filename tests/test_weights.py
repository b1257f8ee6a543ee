"""Weight files: container, binding by name, errors, random folders (no GPU)."""
import json
import os
import struct

import pytest
import torch

import helpers
from ziglm_b200.config import config_from_dict
from ziglm_b200.engine.model import declare_parameters
from ziglm_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_tensors, storage_dtype,
                                write_random_model, write_safetensors)

CPU = torch.device("cpu")


def test_container_round_trip_with_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    back = load_file(p)                                   # the package reads what the library wrote
    for k in t:
        assert torch.equal(back[k], t[k])
    q = str(tmp_path / "y.safetensors")
    save_file(t, q)
    f = SafetensorsFile(q)                                # and the library reads what the package wrote
    assert sorted(f.names()) == ["a", "b", "c"]
    assert f.info("b") == ("BF16", (7,))
    for k in t:
        assert torch.equal(f.tensor(k), t[k])


def _write_raw(path, header: dict, data: bytes, hlen=None):
    raw = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw) if hlen is None else hlen))
        f.write(raw)
        f.write(data)


def test_container_errors(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    _write_raw(p, {}, b"", hlen=1 << 40)
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 4)); f.write(b"[1] ")
    with pytest.raises(SafetensorsError, match="JSON object"):
        SafetensorsFile(p)
    _write_raw(p, {"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8)     # truncated
    with pytest.raises(SafetensorsError, match="data_offsets"):
        SafetensorsFile(p)
    _write_raw(p, {"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}, b"\0" * 16)    # size mismatch
    with pytest.raises(SafetensorsError, match="data_offsets"):
        SafetensorsFile(p)
    _write_raw(p, {"a": {"dtype": "Q4_0", "shape": [4], "data_offsets": [0, 2]}}, b"\0" * 2)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="does not exist"):
        SafetensorsFile(str(tmp_path / "nope.safetensors"))


@pytest.mark.parametrize("name", ["A", "B"])
def test_random_folder_loads_and_is_reproducible(tmp_path, name):
    cfg = helpers.CONFIGS[name]
    c = config_from_dict(cfg)
    f1 = helpers.make_folder(tmp_path / "one", cfg, 11, torch.bfloat16, norm_jitter=0.1)
    f2 = helpers.make_folder(tmp_path / "two", cfg, 11, torch.bfloat16, norm_jitter=0.1)
    f3 = helpers.make_folder(tmp_path / "three", cfg, 12, torch.bfloat16, norm_jitter=0.1)
    declared = declare_parameters(c.model_spec())
    a = load_tensors(f1, declared, torch.bfloat16, CPU)
    b = load_tensors(f2, declared, torch.bfloat16, CPU)
    d = load_tensors(f3, declared, torch.bfloat16, CPU)
    assert set(a) == set(declared)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], d[k]) for k in a)
    assert all(t.dtype == torch.bfloat16 for t in a.values())
    w = a["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.004
    n = a["model.norm.weight"].float()
    assert abs(n.mean().item() - 1.0) < 0.1 and n.std().item() > 0.02        # 1 + N(0, 0.1)
    assert config_from_dict(json.load(open(os.path.join(f1, "config.json")))) == c
    assert ("lm_head.weight" in a) == (not c.tie_word_embeddings)
    assert ("model.layers.0.self_attn.q_proj.bias" in a) == c.attention_bias


def _normal_value_scalar(key: int, i: int):
    """One value of the random fill, written out step by step with float32 scalars (what the library's NumPy
    routine and its kernel compute for element i of the tensor with this key)."""
    import math
    import numpy as np
    f = np.float32
    M = (1 << 64) - 1
    x = (key + i + 0x9E3779B97F4A7C15) & M
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & M
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & M
    h = x ^ (x >> 31)
    n, b = (h >> 40) + 1, (h >> 16) & 0xFFFFFF
    e = n.bit_length() - 1
    m = f(n) * f(2.0 ** -e)
    if m > f(1.41421354):
        m, e = m * f(0.5), e + 1
    s = (m + f(-1.0)) / (m + f(1.0))
    s2 = s * s
    p = f(1.11111111e-1)
    for c in (1.42857143e-1, 0.2, 3.33333333e-1, 1.0):
        p = p * s2 + f(c)
    ln_u = f(e - 24) * f(0.693147182) + (f(2.0) * s) * p
    r = np.sqrt(f(-2.0) * ln_u)
    octant, rem = b >> 21, b & 0x1FFFFF
    xx = f((0x200000 - rem) if octant & 1 else rem) * f(3.74507039e-7)
    x2 = xx * xx
    if octant in (1, 2, 5, 6):
        p = f(2.75573192e-6)
        for c in (-1.98412698e-4, 8.33333333e-3, -1.66666667e-1, 1.0):
            p = p * x2 + f(c)
        c = xx * p
    else:
        p = f(-2.75573192e-7)
        for c in (2.48015873e-5, -1.38888889e-3, 4.16666667e-2, -0.5, 1.0):
            p = p * x2 + f(c)
        c = p
    if octant in (2, 3, 4, 5):
        c = -c
    z = r * c
    # what the steps approximate: sqrt(-2 ln u1) cos(2 pi u2)
    exact = math.sqrt(-2.0 * math.log(n / 2.0 ** 24)) * math.cos(2.0 * math.pi * b / 2.0 ** 24)
    assert abs(float(z) - exact) < 2e-6 * max(1.0, abs(exact))
    return z


def test_random_values_are_a_function_of_seed_name_and_element():
    """Any element of any tensor of a random model can be regenerated alone."""
    import numpy as np
    from ziglm_b200.weights.random_init import normal_values, random_tensor, tensor_key
    from ziglm_b200.parts.base import ParamDecl
    key = tensor_key(11, "model.layers.0.self_attn.q_proj.weight")
    z = normal_values(key, 0, 5000)
    assert z.dtype == np.float32 and np.isfinite(z).all()
    for i in (0, 1, 2, 77, 4999):
        assert _normal_value_scalar(key, i) == z[i]
    assert np.array_equal(normal_values(key, 1234, 100), z[1234:1334])            # a slice needs no other element
    assert not np.array_equal(normal_values(tensor_key(12, "model.layers.0.self_attn.q_proj.weight"), 0, 100), z[:100])
    assert not np.array_equal(normal_values(tensor_key(11, "model.layers.1.self_attn.q_proj.weight"), 0, 100), z[:100])
    big = normal_values(key, 0, 400000).astype(np.float64)
    assert abs(big.mean()) < 0.01 and abs(big.std() - 1.0) < 0.01
    assert abs((big ** 3).mean()) < 0.03 and abs((big ** 4).mean() - 3.0) < 0.1 and np.abs(big).max() > 4.0
    # a tensor is mean + std * z in float32, rounded to its storage type
    t = random_tensor("model.layers.0.self_attn.q_proj.weight", ParamDecl((50, 100)), 11, torch.bfloat16, CPU, std=0.02)
    want = torch.from_numpy(np.float32(0.0) + np.float32(0.02) * z).to(torch.bfloat16).view(50, 100)
    assert torch.equal(t, want)
    n = random_tensor("model.norm.weight", ParamDecl((64,), init="ones"), 11, torch.float32, CPU, norm_jitter=0.1)
    zn = normal_values(tensor_key(11, "model.norm.weight"), 0, 64)
    assert torch.equal(n, torch.from_numpy(np.float32(1.0) + np.float32(0.1) * zn))
    assert torch.equal(random_tensor("x", ParamDecl((8,), init="ones"), 1, torch.float32, CPU), torch.ones(8))


def test_storage_types():
    assert storage_dtype("BF16", "float", torch.bfloat16) == torch.bfloat16
    assert storage_dtype("F16", "float", torch.bfloat16) == torch.bfloat16
    assert storage_dtype("F32", "float", torch.bfloat16) == torch.float32      # stored in 32-bit: stays so
    assert storage_dtype("BF16", "float", torch.float32) == torch.float32
    assert storage_dtype("I64", "int", torch.bfloat16) == torch.int32


def test_32bit_tensors_stay_32bit_in_a_bfloat16_run(tmp_path):
    cfg = helpers.TINY_A
    c = config_from_dict(cfg)
    folder = helpers.make_folder(tmp_path, cfg, 5, torch.bfloat16)
    from safetensors.torch import load_file, save_file
    w = load_file(os.path.join(folder, "model.safetensors"))
    w["model.norm.weight"] = w["model.norm.weight"].float()
    save_file(w, os.path.join(folder, "model.safetensors"))
    t = load_tensors(folder, declare_parameters(c.model_spec()), torch.bfloat16, CPU)
    assert t["model.norm.weight"].dtype == torch.float32
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16
    t32 = load_tensors(folder, declare_parameters(c.model_spec()), torch.float32, CPU)
    assert all(v.dtype == torch.float32 for v in t32.values())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = helpers.TINY_B
    c = config_from_dict(cfg)
    folder = helpers.make_folder(tmp_path, cfg, 5, torch.float32)
    from safetensors.torch import load_file, save_file
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["lm_head.weight"]
    w["model.layers.7.extra.weight"] = torch.zeros(2)
    w["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 96)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)      # a known non-parameter: ignored
    w["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    save_file(w, path)
    with pytest.raises(WeightError) as e:
        load_tensors(folder, declare_parameters(c.model_spec()), torch.float32, CPU)
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert len(err.wrong) == 2
    msg = str(err)
    assert "expected [32, 96], found [64, 96]" in msg and "model.norm.weight" in msg and "floating" in msg
    assert "missing (2)" in msg and "unexpected (1)" in msg


def test_tied_model_refuses_a_separate_head(tmp_path):
    cfg = helpers.TINY_A
    c = config_from_dict(cfg)
    folder = helpers.make_folder(tmp_path, cfg, 5, torch.float32)
    from safetensors.torch import load_file, save_file
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    w["lm_head.weight"] = torch.zeros(256, 64)
    save_file(w, path)
    with pytest.raises(WeightError) as e:
        load_tensors(folder, declare_parameters(c.model_spec()), torch.float32, CPU)
    assert e.value.unexpected == ["lm_head.weight"]


def test_sharded_folder(tmp_path):
    cfg = helpers.TINY_A
    c = config_from_dict(cfg)
    folder = helpers.make_folder(tmp_path, cfg, 5, torch.float32)
    from safetensors.torch import load_file, save_file
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    names = sorted(w)
    half = len(names) // 2
    save_file({k: w[k] for k in names[:half]}, os.path.join(folder, "model-00001-of-00002.safetensors"))
    save_file({k: w[k] for k in names[half:]}, os.path.join(folder, "model-00002-of-00002.safetensors"))
    os.unlink(path)
    idx = {"weight_map": {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                          for i, k in enumerate(names)}}
    json.dump(idx, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    t = load_tensors(folder, declare_parameters(c.model_spec()), torch.float32, CPU)
    assert all(torch.equal(t[k], w[k]) for k in names)


def test_folder_without_weights(tmp_path):
    with pytest.raises(SafetensorsError, match="neither"):
        load_tensors(str(tmp_path), {}, torch.float32, CPU)
