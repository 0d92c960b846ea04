"""Tuning database and auto-tuner (counterparts of TuningDatabase.swift:15-290 and AutoTuner.swift:225-764).

The database half needs no GPU: records are merged as JSON documents in the file format, saved, reloaded, imported,
pruned. The tuner half measures real launches and checks that compiled executables pick the stored configuration up.
"""
import json
import os
import time

import numpy as np
import pytest

from metalhlo_b200 import capi

SWIFT_EPOCH = 978307200.0  # Swift's JSONEncoder writes dates as seconds since 2001-01-01


def record(op, rows, hidden, dtype="bf16", device="NVIDIA B200", threads=256, vecs=2, ctas=4, age_days=0.0):
    key = {"opType": op, "shapes": [[rows, hidden]], "dtype": dtype, "deviceID": device}
    result = {"bestConfig": {"tileM": 0, "tileN": 0, "tileK": 0, "stages": 0, "threads": threads, "vectorsPerThread": vecs, "ctasPerSM": ctas},
              "measuredTime": 1.25e-4, "gflops": 0, "gbytesPerSecond": 4200.5, "configsTried": 17,
              "timestamp": time.time() - age_days * 86400 - SWIFT_EPOCH}
    return key, result


def document(*pairs):
    entries = []
    for k, r in pairs:
        entries += [k, r]
    return {"version": 1, "entries": entries, "savedAt": time.time() - SWIFT_EPOCH}


def test_store_save_reload_round_trip(tmp_path):
    path = str(tmp_path / "tuning.json")
    capi.tuning.open(path)
    assert capi.tuning.count() == 0
    a, b = record("fused_layer_norm", 32768, 4096), record("fused_softmax", 512, 1024, dtype="f32", threads=128, vecs=4, ctas=0)
    assert capi.tuning.merge(document(a, b)) == 2
    assert capi.tuning.count() == 2
    capi.tuning.save()
    on_disk = json.load(open(path))
    assert on_disk["version"] == 1 and len(on_disk["entries"]) == 4  # alternating key, value
    keys = on_disk["entries"][0::2]
    assert {k["opType"] for k in keys} == {"fused_layer_norm", "fused_softmax"}
    # reload from disk into a fresh database object
    capi.tuning.open(str(tmp_path / "other.json"))
    assert capi.tuning.count() == 0
    capi.tuning.open(path)
    assert capi.tuning.count() == 2
    got = capi.tuning.to_dict()
    by_op = {k["opType"]: r for k, r in zip(got["entries"][0::2], got["entries"][1::2])}
    assert by_op["fused_layer_norm"]["bestConfig"]["threads"] == 256
    assert by_op["fused_layer_norm"]["bestConfig"]["ctasPerSM"] == 4
    assert by_op["fused_softmax"]["bestConfig"]["vectorsPerThread"] == 4
    assert by_op["fused_softmax"]["configsTried"] == 17
    assert abs(by_op["fused_softmax"]["gbytesPerSecond"] - 4200.5) < 1e-6


def test_existing_keys_win_unless_overwrite(tmp_path):
    capi.tuning.open(str(tmp_path / "t.json"))
    assert capi.tuning.merge(document(record("fused_rms_norm", 64, 512, threads=64))) == 1
    assert capi.tuning.merge(document(record("fused_rms_norm", 64, 512, threads=128))) == 0
    assert capi.tuning.to_dict()["entries"][1]["bestConfig"]["threads"] == 64
    assert capi.tuning.merge(document(record("fused_rms_norm", 64, 512, threads=128)), overwrite=True) == 1
    assert capi.tuning.to_dict()["entries"][1]["bestConfig"]["threads"] == 128
    # a different device name is a different key
    assert capi.tuning.merge(document(record("fused_rms_norm", 64, 512, device="other GPU"))) == 1
    assert capi.tuning.count() == 2


def test_import_prune_and_clear(tmp_path):
    src = str(tmp_path / "src.json")
    capi.tuning.open(src)
    capi.tuning.merge(document(record("fused_layer_norm", 8, 256, age_days=45), record("fused_layer_norm", 16, 256, age_days=1)))
    capi.tuning.save()
    capi.tuning.open(str(tmp_path / "dst.json"))
    capi.tuning.merge(document(record("fused_layer_norm", 16, 256, threads=32)))
    assert capi.tuning.import_file(src) == 1          # the 16 x 256 entry is already there
    assert capi.tuning.count() == 2
    assert capi.tuning.prune(30) == 1                 # the 45-day-old entry goes
    assert capi.tuning.count() == 1
    capi.tuning.clear()
    assert capi.tuning.count() == 0


def test_malformed_documents_are_rejected(tmp_path):
    capi.tuning.open(str(tmp_path / "t.json"))
    with pytest.raises(capi.MetalHLOError):
        capi.tuning.merge({"version": 1, "entries": [{"opType": "x"}]})  # odd number of items
    rc = capi.lib.mhlo_b200_tuning_merge_json(b'{"entries": [', False, None)
    assert rc == 3  # MHLO_ERROR_PARSE_FAILED
    # a corrupt file on disk is ignored, the database starts empty (the reference prints a warning and starts fresh)
    bad = tmp_path / "bad.json"
    bad.write_text("{ not json")
    capi.tuning.open(str(bad))
    assert capi.tuning.count() == 0


@pytest.mark.gpu
def test_tuner_measures_and_executables_use_the_record(tmp_path):
    import torch

    import oracle
    from metalhlo_b200 import modules
    from parity import assert_close

    capi.tuning.open(str(tmp_path / "gpu.json"))
    client = capi.Client()
    rows, hidden = 4096, 2048
    rec = capi.tuning.tune_row_kernel(client, "fused_layer_norm", capi.BF16, rows, hidden)
    assert rec["configsTried"] >= 4 and rec["measuredTime"] > 0
    assert rec["gbytesPerSecond"] > 1000, rec     # 32 MB in + out: far above 1 TB/s on this GPU even with a poor configuration
    doc = capi.tuning.to_dict()
    key = doc["entries"][0]
    assert key == {"opType": "fused_layer_norm", "shapes": [[rows, hidden]], "dtype": "bf16", "deviceID": client.device_name}
    # force a non-default record so that the executable provably takes the database's configuration
    forced = document(({**key}, {**doc["entries"][1], "bestConfig": {**doc["entries"][1]["bestConfig"], "threads": 256, "vectorsPerThread": 1, "ctasPerSM": 2}}))
    capi.tuning.merge(forced, overwrite=True)
    body, ret = modules.layer_norm_text("%arg0", [rows, hidden], "bf16", gamma="%arg1", beta="%arg2")
    full, vec = modules.tt([rows, hidden], "bf16"), modules.tt([hidden], "bf16")
    text = modules.func([full, vec, vec], [full], body.rstrip("\n"), ret)
    exe = client.compile(text, opt_level=3)
    assert "fused_layer_norm [tuned]" in exe.steps
    g = torch.Generator().manual_seed(0)
    x = torch.randn(rows, hidden, generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    beta = (0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    out, = exe.execute([client.buffer(t) for t in (x, gamma, beta)])
    assert_close(out.to_numpy().astype(np.float64), oracle.layer_norm(x, gamma, beta), 2e-2, "tuned layer_norm")
    capi.tuning.save()
    assert os.path.getsize(str(tmp_path / "gpu.json")) > 100


def contraction_records():
    gemm_key = {"opType": "dot_general", "shapes": [[1, 4096, 768], [1, 768, 3072], [1, 0, 0]], "dtype": "f16", "deviceID": "NVIDIA B200"}
    gemm = {"bestConfig": {"tileM": 256, "tileN": 256, "tileK": 64, "stages": 5, "threads": 0, "vectorsPerThread": 0, "ctasPerSM": 0,
                           "ctaGroup": 2, "tileOrder": 0},
            "measuredTime": 2.4e-5, "gflops": 805000.0, "gbytesPerSecond": 0, "configsTried": 11, "timestamp": time.time() - SWIFT_EPOCH}
    attn_key = {"opType": "fused_scaled_dot_product_attention", "shapes": [[4, 12, 1024, 64], [4, 12, 1024, 64], [1, 1]], "dtype": "f16",
                "deviceID": "NVIDIA B200"}
    attn = {"bestConfig": {"tileM": 0, "tileN": 0, "tileK": 0, "stages": 0, "threads": 0, "vectorsPerThread": 0, "ctasPerSM": 0, "ctaGroup": 0,
                           "tileOrder": 2},
            "measuredTime": 2.7e-5, "gflops": 240000.0, "gbytesPerSecond": 0, "configsTried": 3, "timestamp": time.time() - SWIFT_EPOCH}
    return (gemm_key, gemm), (attn_key, attn)


def test_contraction_records_round_trip_with_their_knobs(tmp_path):
    """Records of the tensor-core GEMM (tile width, ring depth, CTA group) and of the attention kernel (tile order) keep
    every field through merge -> save -> reload; records written before those fields existed read as "library default"."""
    path = str(tmp_path / "contractions.json")
    capi.tuning.open(path)
    g, a = contraction_records()
    old_style = record("dot_general", 8, 8)  # no ctaGroup / tileOrder members
    assert capi.tuning.merge(document(g, a, old_style)) == 3
    capi.tuning.save()
    capi.tuning.open(str(tmp_path / "empty.json"))
    capi.tuning.open(path)
    got = capi.tuning.to_dict()
    by_key = {json.dumps(k, sort_keys=True): r for k, r in zip(got["entries"][0::2], got["entries"][1::2])}
    gr, ar = by_key[json.dumps(g[0], sort_keys=True)], by_key[json.dumps(a[0], sort_keys=True)]
    assert (gr["bestConfig"]["tileN"], gr["bestConfig"]["stages"], gr["bestConfig"]["ctaGroup"]) == (256, 5, 2)
    assert abs(gr["gflops"] - 805000.0) < 1e-3 and gr["configsTried"] == 11
    assert ar["bestConfig"]["tileOrder"] == 2 and ar["bestConfig"]["ctaGroup"] == 0
    orr = by_key[json.dumps(old_style[0], sort_keys=True)]
    assert orr["bestConfig"]["ctaGroup"] == 0 and orr["bestConfig"]["tileOrder"] == 0


@pytest.mark.gpu
def test_gemm_tuner_measures_and_executables_use_the_record(tmp_path):
    import torch

    import oracle
    from metalhlo_b200 import modules
    from parity import assert_close

    capi.tuning.open(str(tmp_path / "gemm.json"))
    client = capi.Client()
    m, k, n = 2048, 768, 1024
    rec = capi.tuning.tune_gemm(client, capi.F16, 1, m, n, k)
    assert rec["configsTried"] >= 8 and rec["measuredTime"] > 0 and rec["gflops"] > 50_000, rec
    doc = capi.tuning.to_dict()
    key = doc["entries"][0]
    assert key == {"opType": "dot_general", "shapes": [[1, m, k], [1, k, n], [1, 0, capi.F16]], "dtype": "f16", "deviceID": client.device_name}
    tx, tw, to = modules.tt((m, k), "f16"), modules.tt((k, n), "f16"), modules.tt((m, n), "f16")
    text = f"func.func @main(%x: {tx}, %w: {tw}) -> {to} {{\n  %0 = stablehlo.dot_general %x, %w, contracting_dims = [1] x [0] : ({tx}, {tw}) -> {to}\n  return %0 : {to}\n}}\n"
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(m, k, generator=g) / k ** 0.5).to(torch.float16)
    w = torch.randn(k, n, generator=g).to(torch.float16)
    want = oracle.gemm(x, w)
    results = []
    # force two different non-default records in turn: the executable provably launches what the database holds
    for cfg in ({"tileN": 128, "stages": 3, "ctaGroup": 1}, {"tileN": 256, "stages": 4, "ctaGroup": 2}):
        forced = {**doc["entries"][1], "bestConfig": {**doc["entries"][1]["bestConfig"], **cfg}}
        capi.tuning.merge(document((key, forced)), overwrite=True)
        exe = client.compile(text, opt_level=3, caching=False)
        assert exe.steps == ["dot_general [tuned]"], exe.steps
        out, = exe.execute([client.buffer(x), client.buffer(w)])
        got = out.to_numpy()
        assert_close(got.astype(np.float64), want, 2e-2, f"tuned gemm {cfg}")
        results.append(got)
    assert np.array_equal(results[0].view(np.uint16), results[1].view(np.uint16))
    # a record that holds the library's own choice leaves the step untuned
    capi.tuning.merge(document((key, {**doc["entries"][1], "bestConfig": {k_: 0 for k_ in doc["entries"][1]["bestConfig"]}})), overwrite=True)
    assert client.compile(text, opt_level=3, caching=False).steps == ["dot_general"]


@pytest.mark.gpu
def test_attention_tuner_measures_and_executables_use_the_record(tmp_path):
    import torch

    import oracle
    from op_cases import attention_text
    from parity import assert_close

    capi.tuning.open(str(tmp_path / "attn.json"))
    client = capi.Client()
    b, h, s, d = 2, 4, 512, 64
    rec = capi.tuning.tune_attention(client, capi.BF16, b, h, s, s, d, causal=True)
    assert rec["configsTried"] == 3 and rec["measuredTime"] > 0 and rec["gflops"] > 1000, rec
    doc = capi.tuning.to_dict()
    key = doc["entries"][0]
    assert key["opType"] == "fused_scaled_dot_product_attention" and key["shapes"] == [[b, h, s, d], [b, h, s, d], [1, 0]]
    text, qshape = attention_text(b, h, s, d, "bf16", True, "BHSD")
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(*qshape, generator=g).to(torch.bfloat16) for _ in range(3))
    want = oracle.attention(q, k, v, 1 / d ** 0.5, causal=True)
    mag = oracle.attention(q, k, v.abs(), 1 / d ** 0.5, causal=True)
    outs = []
    for order in (1, 2):
        forced = {**doc["entries"][1], "bestConfig": {**doc["entries"][1]["bestConfig"], "tileOrder": order}}
        capi.tuning.merge(document((key, forced)), overwrite=True)
        exe = client.compile(text, opt_level=3, caching=False)
        assert "fused_scaled_dot_product_attention [tuned]" in exe.steps, exe.steps
        out, = exe.execute([client.buffer(t) for t in (q, k, v)])
        got = out.to_numpy()
        assert_close(got.astype(np.float64), want, 2e-2, f"tile order {order}", magnitude=mag)
        outs.append(got)
    assert np.array_equal(outs[0].view(np.uint16), outs[1].view(np.uint16))  # the order of the tiles does not change any row's arithmetic
