"""Checkpoint ingest (safetensors / torch-pickle directories) on CPU: format parsing, the reference's key matching
rule, refusal of anything executable in a pickle, and the copy into the training step's parameter structure."""
import io
import json
import os
import pickle
import struct
import zipfile
from collections import OrderedDict

import numpy as np
import pytest
import torch

from cacti_b200 import ingest
from cacti_b200.llama_step import LlamaShape, init_weights, zeros_like_params

CFG = LlamaShape(layers=2, d_model=16, heads=2, head_dim=8, ffn=24, vocab=32, seq=8)


def hf_state(P):
    """The parameter structure under the names a Hugging Face LLaMA checkpoint uses."""
    sd = OrderedDict()
    sd["model.embed_tokens.weight"] = P["embed"]
    for i, L in enumerate(P["layers"]):
        pre = f"model.layers.{i}."
        sd[pre + "self_attn.q_proj.weight"] = L["q"]
        sd[pre + "self_attn.k_proj.weight"] = L["k"]
        sd[pre + "self_attn.v_proj.weight"] = L["v"]
        sd[pre + "self_attn.o_proj.weight"] = L["o"]
        sd[pre + "mlp.gate_proj.weight"] = L["gate"]
        sd[pre + "mlp.down_proj.weight"] = L["down"]
        sd[pre + "mlp.up_proj.weight"] = L["up"]
        sd[pre + "input_layernorm.weight"] = L["pre_norm"]
        sd[pre + "post_attention_layernorm.weight"] = L["post_norm"]
    sd["model.norm.weight"] = P["head_norm"]
    sd["lm_head.weight"] = P["lm_head"]
    return sd


def write_safetensors(path, tensors, metadata=True):
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {"format": "pt"}
    for name, t in tensors.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.numel() else b""
        tag = {torch.float16: "F16", torch.float32: "F32", torch.bfloat16: "BF16", torch.int32: "I32"}[t.dtype]
        header[name] = {"dtype": tag, "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def same(P, Q):
    a = dict(ingest_flat(P))
    b = dict(ingest_flat(Q))
    return all(torch.equal(a[k], b[k]) for k in a) and a.keys() == b.keys()


def ingest_flat(P):
    yield from ((k, v) for k, v in P.items() if k != "layers")
    for i, L in enumerate(P["layers"]):
        yield from ((f"layers.{i}.{k}", v) for k, v in L.items())


@pytest.fixture(scope="module")
def weights():
    P = init_weights(CFG, torch.device("cpu"), seed=3)
    for L in P["layers"]:                      # distinct norm gains so a swapped match would show
        L["pre_norm"].add_(torch.randn(CFG.d_model).half() * 0.1)
        L["post_norm"].add_(torch.randn(CFG.d_model).half() * 0.1)
    return P


def test_safetensors_single_file(tmp_path, weights):
    sd = hf_state(weights)
    write_safetensors(tmp_path / "model.safetensors", sd)
    d = ingest.TensorsDir.open(tmp_path)
    assert d.clone_keys() == set(sd) and d.serial_key == list(sd)
    tag, shape, view = d.get("model.layers.1.mlp.up_proj.weight")
    assert tag == "F16" and shape == (CFG.ffn, CFG.d_model)
    assert bytes(view) == weights["layers"][1]["up"].view(torch.uint8).numpy().tobytes()
    Q = zeros_like_params(weights)
    m = ingest.load_llama(d, Q)
    assert same(weights, Q)
    assert m["head_norm"] == "model.norm.weight" and m["layers.1.pre_norm"] == "model.layers.1.input_layernorm.weight"
    d.close()


def test_safetensors_shards_and_errors(tmp_path, weights):
    sd = list(hf_state(weights).items())
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", OrderedDict(sd[11:]))
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", OrderedDict(sd[:11]), metadata=False)
    d = ingest.TensorsDir.open(tmp_path)
    assert [os.path.basename(p) for p in d.model_paths] == ["model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"]
    Q = zeros_like_params(weights)
    ingest.load_llama(d, Q)
    assert same(weights, Q)
    # a name present in two shards
    write_safetensors(tmp_path / "model-00003-of-00003.safetensors", OrderedDict(sd[:1]))
    with pytest.raises(ingest.IngestError) as e:
        ingest.TensorsDir.open(tmp_path)
    assert e.value.kind == "DuplicateName"
    with pytest.raises(ingest.IngestError) as e:
        ingest.TensorsDir.open(tmp_path / "nothing_here")
    assert e.value.kind == "Path"
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "model.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ingest.IngestError) as e:
        ingest.TensorsDir.open(bad)
    assert e.value.kind == "TensorsDict"
    (bad / "model.safetensors").write_bytes(struct.pack("<Q", 60) + json.dumps(
        {"w": {"dtype": "F16", "shape": [4], "data_offsets": [0, 9000]}}).encode().ljust(60))
    with pytest.raises(ingest.IngestError):
        ingest.TensorsDir.open(bad)
    # a shape that disagrees with the byte range is caught at get()
    (bad / "model.safetensors").write_bytes(struct.pack("<Q", 64) + json.dumps(
        {"w": {"dtype": "F16", "shape": [4], "data_offsets": [0, 6]}}).encode().ljust(64) + b"\0" * 6)
    with pytest.raises(ingest.IngestError):
        ingest.TensorsDir.open(bad).get("w")


def test_model_shape_or_dtype_mismatch(tmp_path, weights):
    sd = hf_state(weights)
    sd["lm_head.weight"] = sd["lm_head.weight"].float()
    write_safetensors(tmp_path / "model.safetensors", sd)
    with pytest.raises(ingest.IngestError):
        ingest.load_llama(ingest.TensorsDir.open(tmp_path), zeros_like_params(weights))
    del sd["model.norm.weight"]
    write_safetensors(tmp_path / "model.safetensors", sd)
    with pytest.raises(ingest.IngestError) as e:
        ingest.load_llama(ingest.TensorsDir.open(tmp_path), zeros_like_params(weights))
    assert e.value.kind == "Path"


def test_matcher_rule():
    """Ints match a whole token, strings a substring; rules take keys in order and never share one."""
    m = ingest.CellMatcher()
    m.insert((1, "attn", "q_proj"), "q1")
    m.insert((1, "layernorm"), "ln1")
    m.insert("norm", "final")
    keys = {"model.layers.1.self_attn.q_proj.weight", "model.layers.11.self_attn.q_proj.weight", "model.norm.weight",
            "model.layers.1.input_layernorm.weight", "unrelated"}
    got = dict((t, k) for k, t in m.match_(keys))
    assert got == {"q1": "model.layers.1.self_attn.q_proj.weight", "ln1": "model.layers.1.input_layernorm.weight",
                   "final": "model.norm.weight"}


def test_pickle_dir(tmp_path, weights):
    sd = hf_state(weights)
    items = list(sd.items())
    torch.save(OrderedDict(items[:9]), tmp_path / "pytorch_model-00001-of-00002.bin")
    torch.save(OrderedDict(items[9:]), tmp_path / "pytorch_model-00002-of-00002.bin")
    d = ingest.PickleDir.open(tmp_path)
    assert d.clone_keys() == set(sd)
    tag, shape, view = d.get("model.layers.0.self_attn.k_proj.weight")
    assert (tag, shape) == ("F16", (CFG.d_model, CFG.d_model))
    assert bytes(view) == weights["layers"][0]["k"].view(torch.uint8).numpy().tobytes()
    Q = zeros_like_params(weights)
    ingest.load_llama(d, Q)
    assert same(weights, Q)


def test_pickle_views_share_a_storage_and_strided_is_refused(tmp_path):
    base = torch.arange(64, dtype=torch.float32)
    one = tmp_path / "a"
    one.mkdir()
    torch.save(OrderedDict(lo=base[:16].view(4, 4), hi=base[32:].view(2, 16)), one / "pytorch_model.bin")
    d = ingest.PickleDir.open(one)
    assert np.frombuffer(d.get("hi")[2], np.float32).tolist() == list(range(32, 64))
    assert np.frombuffer(d.get("lo")[2], np.float32).tolist() == list(range(16))
    two = tmp_path / "b"
    two.mkdir()
    torch.save(OrderedDict(t=base.view(8, 8).t()), two / "pytorch_model.bin")
    with pytest.raises(ingest.IngestError) as e:
        ingest.PickleDir.open(two)
    assert e.value.kind == "PickleFile" and "strided" in str(e.value)


class _Boom:
    def __reduce__(self):
        return (os.system, ("touch " + os.environ["CACTI_B200_INGEST_CANARY"],))


def test_pickle_is_interpreted_never_executed(tmp_path):
    canary = tmp_path / "canary"
    os.environ["CACTI_B200_INGEST_CANARY"] = str(canary)
    payload = pickle.dumps(OrderedDict(w=_Boom()), protocol=2)
    with zipfile.ZipFile(tmp_path / "pytorch_model.bin", "w", zipfile.ZIP_STORED) as z:
        z.writestr("archive/data.pkl", payload)
    with pytest.raises(ingest.IngestError) as e:
        ingest.PickleDir.open(tmp_path)
    assert e.value.kind == "PickleFile" and not canary.exists()
    (tmp_path / "pytorch_model.bin").write_bytes(b"not a zip")
    with pytest.raises(ingest.IngestError):
        ingest.PickleDir.open(tmp_path)


class _Stor:            # stands for a storage; written as a persistent id, as torch.save does
    def __init__(self, numel):
        self.numel = numel


class _Rec:             # pickles as a call of torch._utils._rebuild_tensor_v2 with arguments of the test's choosing
    def __init__(self, *args):
        self.args = args

    def __reduce__(self):
        import torch._utils
        return (torch._utils._rebuild_tensor_v2, self.args)


def _crafted_archive(path, record, storage_bytes=64 * 2):
    import io

    class P(pickle.Pickler):
        def persistent_id(self, obj):
            if isinstance(obj, _Stor):
                return ("storage", torch.HalfStorage, "0", "cpu", obj.numel)
            return None

    buf = io.BytesIO()
    P(buf, protocol=2).dump(OrderedDict(w=record))
    with zipfile.ZipFile(path, "w", zipfile.ZIP_STORED) as z:
        z.writestr("archive/data.pkl", buf.getvalue())
        # the storage starts on a 64-byte boundary of the archive, as torch.save writes it (padding in the extra field)
        info = zipfile.ZipInfo("archive/data/0")
        pad = -(z.fp.tell() + 30 + len(info.filename) + 4) % 64
        info.extra = struct.pack("<HH", 0x4246, pad) + bytes(pad)
        z.writestr(info, bytes(storage_bytes))


@pytest.mark.parametrize("what,args", [
    ("negative offset", (_Stor(64), -8, (4, 4), (4, 1))),
    ("negative dimension", (_Stor(64), 0, (-4, 4), (4, 1))),
    ("offset past the storage", (_Stor(64), 60, (4, 4), (4, 1))),
    ("first argument is not a storage", (7, 0, (4, 4), (4, 1))),
    ("non-integer dimension", (_Stor(64), 0, (4.0, 4), (4, 1))),
    ("shape is not a sequence", (_Stor(64), 0, 16, (1,))),
])
def test_pickle_records_with_hostile_numbers_are_refused(tmp_path, what, args):
    """Offsets, dimensions and the storage reference come from the file: a crafted record must end in IngestError,
    never in a slice of other bytes of the archive or in a Python exception of another kind."""
    _crafted_archive(tmp_path / "pytorch_model.bin", _Rec(*args))
    with pytest.raises(ingest.IngestError) as e:
        ingest.PickleDir.open(tmp_path)
    assert e.value.kind == "PickleFile", what


def test_pickle_record_well_formed_by_hand(tmp_path):
    _crafted_archive(tmp_path / "pytorch_model.bin", _Rec(_Stor(64), 16, (4, 4), (4, 1)))
    d = ingest.PickleDir.open(tmp_path)
    assert d.get("w")[1] == (4, 4) and len(bytes(d.get("w")[2])) == 32
