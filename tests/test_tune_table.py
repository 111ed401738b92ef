"""The tuning table: a JSON file written by `python -m ccglib_b200.tune --write` that a plan
consults (CCGLIB_B200_TUNE_TABLE) before its built-in tile model.  Host-side lookup on CPU; the
override itself, with bit-identical results, on the GPU."""
import json

import numpy as np
import pytest

from ccglib_b200 import capi, tune


def _table(tmp_path, entries):
    path = tmp_path / "table.json"
    path.write_text(json.dumps({"format": tune.TABLE_FORMAT, "entries": entries}, indent=1))
    return str(path)


def test_lookup_matches_types_shape_and_buckets(tmp_path):
    key = tune.table_key(capi.FLOAT16, capi.FLOAT32, 6, 512, 768, 1000)
    assert key["k_bucket"] == 11 and key["batch_bucket"] == 3  # 2000 bytes per row, batch 6
    path = _table(tmp_path, [
        dict(tune.table_key(capi.BFLOAT16, capi.FLOAT32, 6, 512, 768, 1000), bn=64, pair=0,
             group_n=2),
        dict(key, bn=256, pair=1, group_n=16, tops=123.4, form="pair, 256 columns", data="random"),
    ])
    assert capi.tune_table_lookup(path, 6, 512, 768, 1000, capi.FLOAT16, capi.FLOAT32) == (256, 1, 16)
    assert capi.tune_table_lookup(path, 8, 512, 768, 1024, capi.FLOAT16, capi.FLOAT32) == (256, 1, 16)
    assert capi.tune_table_lookup(path, 6, 512, 768, 1000, capi.BFLOAT16, capi.FLOAT32) == (64, 0, 2)
    # another shape, another batch bucket, another row-length bucket: no entry
    assert capi.tune_table_lookup(path, 6, 512, 769, 1000, capi.FLOAT16, capi.FLOAT32) is None
    assert capi.tune_table_lookup(path, 9, 512, 768, 1000, capi.FLOAT16, capi.FLOAT32) is None
    assert capi.tune_table_lookup(path, 6, 512, 768, 2000, capi.FLOAT16, capi.FLOAT32) is None
    assert capi.tune_table_lookup(str(tmp_path / "missing.json"), 6, 512, 768, 1000,
                                  capi.FLOAT16, capi.FLOAT32) is None


def test_merge_replaces_the_entry_of_the_same_key(tmp_path):
    path = str(tmp_path / "t.json")
    key = tune.table_key(capi.INT1, capi.INT32, 32, 4096, 4096, 65536)
    tune.merge_into_table(path, dict(key, bn=192, pair=1, group_n=0))
    tune.merge_into_table(path, dict(tune.table_key(capi.INT1, capi.INT32, 1, 64, 64, 256),
                                     bn=128, pair=0, group_n=0))
    tune.merge_into_table(path, dict(key, bn=224, pair=1, group_n=4))
    table = json.load(open(path))
    assert table["format"] == tune.TABLE_FORMAT and len(table["entries"]) == 2
    assert capi.tune_table_lookup(path, 32, 4096, 4096, 65536, capi.INT1, capi.INT32) == (224, 1, 4)


@pytest.mark.gpu
@pytest.mark.parametrize("types", [(capi.FLOAT16, capi.FLOAT32), (capi.INT1, capi.INT32)],
                         ids=["f16", "int1"])
def test_table_entry_overrides_the_model_with_identical_results(tmp_path, monkeypatch, types):
    import torch

    import gpu_util as gu
    import oracle_util as ou
    from test_gpu_gemm import make_inputs

    type_in, type_out = types
    B, M, N, K = 3, 300, 520, 1056
    # compare tile forms only: split-K (which the model would pick for so few tiles) adds the
    # partial sums of the K shares in another order
    monkeypatch.setenv("CCGLIB_B200_SPLITK", "1")
    a, b = make_inputs(61, type_in, B, M, N, K)
    d_a, d_b = gu.dev(a), gu.dev(b)
    c_bytes = B * 2 * M * N * 4

    def run():
        plan = capi.GemmPlan(B, M, N, K, type_in, type_out, variant=capi.BASIC)
        tile = plan.tile
        d_c = gu.dev_empty(c_bytes, 0xEE)
        plan.run(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), gu.stream_handle())
        torch.cuda.synchronize()
        gu.check_device_status()
        plan.close()
        return tile, d_c

    model_tile, c_model = run()
    assert not model_tile["tuned"]
    other_bn = 128 if model_tile["bn"] != 128 else (192 if type_in == capi.INT1 else 256)
    entry = dict(tune.table_key(type_in, type_out, B, M, N, K), bn=other_bn,
                 pair=1 - model_tile["pair"], group_n=3)
    monkeypatch.setenv("CCGLIB_B200_TUNE_TABLE", _table(tmp_path, [entry]))
    tuned_tile, c_tuned = run()
    assert tuned_tile == {"bn": other_bn, "pair": 1 - model_tile["pair"], "group_n": 3,
                          "tuned": True, "split_k": 1}
    # each element still sums its K products in the same order: identical bits
    assert torch.equal(c_model, c_tuned)
    got = gu.host(c_tuned, ou.STORAGE[type_out]).reshape(B, 2, M, N)
    if type_in == capi.INT1:
        assert np.array_equal(got, gu.oracle_batch(type_in, type_out, a, b, B, M, N, K))
    else:
        gu.assert_close_fp64(got, type_in, type_out, a, b, K)
    # the environment still wins over the table
    monkeypatch.setenv("CCGLIB_B200_BN", str(model_tile["bn"]))
    env_tile, _ = run()
    assert env_tile["bn"] == model_tile["bn"]
