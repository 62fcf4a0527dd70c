"""GGUF ingestion on the CPU: the self-contained reader against files written (and re-read) by the `gguf` package."""
import numpy as np
import pytest
import torch

gguf = pytest.importorskip("gguf")

from paramecia_b200 import synth
from paramecia_b200.gguf import GGUFError, GGUFFile, moe_layer_names, moe_layers
from tests.gguf_util import write_layer_gguf


@pytest.mark.parametrize("preset,router", [("q4k_m", "f32"), ("q6k", "f16"), ("q8_0", "bf16")])
def test_reader_matches_gguf_package(tmp_path, preset, router):
    t = synth.make_layer(E=4, k=2, preset=preset, seed=3)
    path = str(tmp_path / "layer.gguf")
    write_layer_gguf(path, t, layer=7, router_dtype=router)
    ref = gguf.GGUFReader(path)
    with GGUFFile(path) as f:
        assert f.version == 3
        assert f.metadata["qwen3next.expert_count"] == 4 and f.meta("qwen3next.expert_used_count") == 2
        assert f.meta("nope", "qwen3next.embedding_length") == 2048
        assert f.metadata["general.architecture"] == "qwen3next"
        assert moe_layers(f) == [7]
        assert len(f.tensors) == len(ref.tensors)
        for rt in ref.tensors:
            info = f.tensors[rt.name]
            assert info.dtype == int(rt.tensor_type)
            assert info.shape == tuple(int(v) for v in reversed(rt.shape.tolist()))
            assert np.array_equal(f.tensor_bytes(rt.name), np.asarray(rt.data).reshape(-1).view(np.uint8))
        names = moe_layer_names(7)
        assert f.tensors[names["gate_exps"]].shape == (4, 512, 2048)
        assert f.tensors[names["down_exps"]].shape == (4, 2048, 512)
        assert np.array_equal(f.tensor_bytes(names["gate_exps"]), t["gate"].numpy())
        assert np.array_equal(f.tensor_bytes(names["sh_down"]), t["shared"]["down"].numpy())


def test_reader_rejects_bad_files(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGML" + b"\0" * 60)
    with pytest.raises(GGUFError):
        GGUFFile(str(p))
    p.write_bytes(b"GGUF" + (9).to_bytes(4, "little") + b"\0" * 16)
    with pytest.raises(GGUFError):
        GGUFFile(str(p))
    t = synth.make_layer(E=2, k=1, preset="q8_0", seed=1, shared=False)
    good = str(tmp_path / "good.gguf")
    write_layer_gguf(good, t)
    data = open(good, "rb").read()
    p.write_bytes(data[:len(data) // 2])   # truncated in the data section
    with GGUFFile(str(p)) as f, pytest.raises(GGUFError):
        f.tensor_bytes("token_embd.weight")
    with GGUFFile(good) as f, pytest.raises(GGUFError):
        f.tensor_bytes("blk.0.missing")
