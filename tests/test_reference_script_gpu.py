"""The reference's own driver script, ``run_nemotron_8b_decode_degradation.py``, run UNCHANGED from ``baseline/_ref`` on
the stand-in model directory (tests/reference_env.py): once with this repository's ``hybrid_quant`` first on the path
(the library's kernels behind the reference's patch functions), once with the reference's package alone (its Triton
kernels), both in child processes.  The two runs must report the same perplexities up to the kernels' rounding."""
import json
import subprocess

import pytest

from tests import reference_env as renv

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not renv.SCRIPT.exists(), reason="baseline/_ref is empty (python baseline/reference.py --from <checkout>)")]

CTX, STEPS = 32, 16


def _run(tmp_path, env, experiments, use_library, tag, extra=()):
    out = tmp_path / "results" / tag / "data" / "degradation.jsonl"
    args = ["--repo", str(env["repo"]), "--dataset", str(env["dataset"]), "--context-length", str(CTX), "--decode-steps", str(STEPS),
            "--checkpoint-steps", f"{STEPS // 2},{STEPS}", "--experiments", experiments, "--kv-group-size", "32", "--progress-every", "8",
            "--output", str(out), *extra]
    res = subprocess.run(renv.script_command(args, use_library=use_library), cwd=tmp_path, env=renv.subprocess_env(tmp_path),
                         capture_output=True, text=True, timeout=1500)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-6000:]
    rows = [json.loads(line) for line in out.read_text().splitlines()]
    assert out.with_suffix(".csv").exists() and (tmp_path / "results" / tag / "figures" / "degradation.png").exists()
    return {r["experiment"]: r for r in rows if r.get("event") == "final"}, rows


def test_reference_script_runs_unchanged_on_the_library(tmp_path):
    env = renv.build(tmp_path)
    finals, rows = _run(tmp_path, env, "baseline,kv_int4,ssm_mx8,ssm_mx8_skip_attn_adjacent,ssm_mx4,both_int4_mx8,both_int4_mx4", True, "ours")
    assert set(finals) == {"baseline", "kv_int4", "ssm_mx8", "ssm_mx8_skip_attn_adjacent", "ssm_mx4", "both_int4_mx8", "both_int4_mx4"}
    base = finals["baseline"]["ppl"]
    assert base > 1.0 and all(f["tokens"] == STEPS for f in finals.values())
    for name, f in finals.items():
        drift = abs(f["ppl"] / base - 1.0)
        print(f"{name}: ppl {f['ppl']:.3f} ({drift * 100:.2f} % from the bf16 run)")
        assert drift < (0.5 if "mx4" in name else 0.1), (name, f["ppl"], base)
    checkpoints = [r for r in rows if r.get("event") == "checkpoint"]
    assert {r["decode_steps"] for r in checkpoints} == {STEPS // 2, STEPS}
    assert all(r["state_backend"] == "mx8_kernel" for r in checkpoints if r["experiment"] == "ssm_mx8")


def test_same_perplexities_as_the_reference_kernels(tmp_path):
    """Deterministic rounding, so both implementations walk the same trajectory: the script's perplexities with the
    library's kernels against the same script with the reference's own Triton kernels."""
    pytest.importorskip("triton")
    env = renv.build(tmp_path)
    exps = "baseline,kv_int4,ssm_mx8,both_int4_mx8"
    ours, _ = _run(tmp_path, env, exps, True, "ours", extra=("--deterministic",))
    theirs, _ = _run(tmp_path, env, exps, False, "reference", extra=("--deterministic",))
    for name in exps.split(","):
        a, b = ours[name]["ppl"], theirs[name]["ppl"]
        print(f"{name}: library {a:.4f}  reference {b:.4f}")
        assert abs(a / b - 1.0) < (1e-6 if name == "baseline" else 2e-2), (name, a, b)
