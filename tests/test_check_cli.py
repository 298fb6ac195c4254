"""The ``check``-compatible command (tests/check_cli.py): argument contract on the CPU, a passing and a failing
comparison of a twin against the evaluator on the GPU."""
import json

import pytest
import torch

from tests import check_cli
from tilefoundry_b200.runtime import AllClose, Equal


def _expect(argv):
    return check_cli.expectations(getattr(check_cli.build_parser().parse_args(["f.py:X", *argv]), "comparison", None))


def test_ordered_comparison_arguments():
    e = _expect(["--out", "output[0]", "--fn", "allclose", "--atol", "1e-2", "--rtol", "2e-2", "--fn", "nan_inf",
                 "--out", "output[1]", "--fn", "equal"])
    assert list(e) == ["output[0]", "output[1]"]
    assert e["output[0]"][0] == AllClose(atol=1e-2, rtol=2e-2) and e["output[0]"][1].name == "nan_inf"
    assert e["output[1]"] == [Equal()]


@pytest.mark.parametrize("argv,msg", [
    ([], "no comparison requested"),
    (["--fn", "equal"], "before any --out"),
    (["--out", "output", "--atol", "1"], "before any --fn"),
    (["--out", "output", "--fn", "allclose", "--atol", "1"], "missing"),
    (["--out", "output", "--fn", "equal", "--atol", "1"], "takes no"),
])
def test_comparison_usage_errors(argv, msg):
    with pytest.raises(ValueError, match=msg):
        _expect(argv)


def test_unknown_subject_is_a_usage_error(capsys):
    assert check_cli.run(["tilefoundry_b200/twins/qwen3_1_7b.py:no_such_thing", "--out", "output", "--fn", "nan_inf"]) == 2
    assert "no 'no_such_thing'" in capsys.readouterr().err
    assert check_cli.run(["nowhere.py:make_twin", "--out", "output", "--fn", "nan_inf"]) == 2


def test_seeded_draws_are_shared_by_both_sides():
    from tilefoundry_b200.authored import qwen3_1_7b as q
    sem = q.build(q.QWEN3_TINY)
    res = check_cli.RandomWeights(sem, torch.Generator().manual_seed(0), {})
    a = res.subtree("layer0").load("w_gate")
    assert res.subtree("layer0").load("w_gate") is a                      # cached: one draw, two readers
    assert a.dtype == torch.bfloat16 and tuple(a.shape) == (1, 256, 512)
    assert abs(float(res.subtree("layer0").load("gamma_in").float().mean()) - 1.0) < 0.05


@pytest.mark.gpu
def test_check_command_passes_and_fails_on_the_gpu(capsys):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    subject = "tilefoundry_b200/twins/qwen3_1_7b.py:make_twin.layer0.mlp"
    ok = check_cli.run([subject, "--inputs", "random", "--out", "output", "--fn", "allclose", "--atol", "2e-2", "--rtol",
                        "2e-2", "--fn", "nan_inf", "--json"])
    rec = json.loads(capsys.readouterr().out)
    assert ok == 0 and rec["passed"] and rec["function"] == "mlp" and rec["outputs"][0]["path"] == "output"
    assert [m["fn"] for m in rec["outputs"][0]["fns"]] == ["allclose", "nan_inf"]
    # a bound that cannot be met must FAIL (the reference's installed-surface tests make the same negative check,
    # tests/installed/models/contract.py:359-370)
    bad = check_cli.run([subject, "--out", "output", "--fn", "max_abs", "--max", "-1"])
    assert bad == 1 and capsys.readouterr().out.rstrip().endswith("FAIL")
    # a function with several outputs and a range to bind
    attn = check_cli.run(["tilefoundry_b200/twins/qwen3_1_7b.py:make_twin.layer0.self_attention", "--dim", "ctx_len=24",
                          "--out", "output[0]", "--fn", "allclose", "--atol", "2e-2", "--rtol", "2e-2",
                          "--out", "output[1]", "--fn", "allclose", "--atol", "2e-2", "--rtol", "2e-2",
                          "--out", "output[2]", "--fn", "allclose", "--atol", "2e-2", "--rtol", "2e-2"])
    out = capsys.readouterr().out
    assert attn == 0 and out.rstrip().endswith("PASS") and "output[2]" in out
    # the range left unbound is a usage error
    assert check_cli.run(["tilefoundry_b200/twins/qwen3_1_7b.py:make_twin.layer0.self_attention", "--out", "output[0]",
                          "--fn", "nan_inf"]) == 2
