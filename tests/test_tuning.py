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
