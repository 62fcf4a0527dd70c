"""Writes a synthetic MoE layer (paramecia_b200.synth.make_layer) as a GGUF file with the tensor names and
metadata keys the reference reads.  Test infrastructure: uses the `gguf` Python package as the writer."""
import numpy as np
import torch


def write_layer_gguf(path, t, layer=0, router_dtype="f32", arch="qwen3next", alt_gate_name=False):
    import gguf
    from gguf import GGMLQuantizationType as T
    from paramecia_b200 import _lib

    def raw(u8: torch.Tensor, dtype: int, *dims):
        rows, cols = dims[:-1], dims[-1]
        return u8.cpu().numpy().reshape(*rows, _lib.row_bytes(dtype, cols)), T(dtype)

    w = gguf.GGUFWriter(path, arch)
    w.add_uint32(f"{arch}.expert_count", t["E"])
    w.add_uint32(f"{arch}.expert_used_count", t["k"])
    w.add_uint32(f"{arch}.embedding_length", t["H"])
    w.add_uint32(f"{arch}.expert_feed_forward_length", t["F"])
    p = f"blk.{layer}"
    E, F, H = t["E"], t["F"], t["H"]
    for name, key, dims in (("ffn_gate_exps", "gate", (E, F, H)), ("ffn_up_exps", "up", (E, F, H)),
                            ("ffn_down_exps", "down", (E, H, F))):
        arr, dt = raw(t[key], t[f"{key}_dtype"], *dims)
        w.add_tensor(f"{p}.{name}.weight", arr, raw_dtype=dt)
    r = t["router_w"].cpu()
    if router_dtype == "blocks":   # the quantised router of make_layer(router_dtype=...)
        arr, dt = raw(t["router_q"], t["router_dtype"], E, H)
        w.add_tensor(f"{p}.ffn_gate_inp.weight", arr, raw_dtype=dt)
    elif router_dtype == "f32":
        w.add_tensor(f"{p}.ffn_gate_inp.weight", r.float().numpy())
    elif router_dtype == "f16":
        w.add_tensor(f"{p}.ffn_gate_inp.weight", r.half().numpy())
    else:
        w.add_tensor(f"{p}.ffn_gate_inp.weight", r.bfloat16().view(torch.uint8).numpy().reshape(E, H * 2), raw_dtype=T.BF16)
    s = t["shared"]
    if s is not None:
        for name, key, dims in (("ffn_gate_shexp", "gate", (F, H)), ("ffn_up_shexp", "up", (F, H)),
                                ("ffn_down_shexp", "down", (H, F))):
            arr, dt = raw(s[key], s[f"{key}_dtype"], *dims)
            w.add_tensor(f"{p}.{name}.weight", arr, raw_dtype=dt)
        gname = f"{p}.ffn_gate_inp_shexp" + ("" if alt_gate_name else ".weight")
        w.add_tensor(gname, s["gate_inp"].cpu().float().numpy())
    w.add_tensor("token_embd.weight", np.zeros((4, 32), np.float32))   # an unrelated tensor in front of nothing
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
