"""The runner environment of the reference's driver script, as far as it goes without a GPU: every import the script
makes resolves (this repository's ``hybrid_quant`` for the two hot paths, the reference's package for the rest, the
matplotlib stand-in), and the stand-in model directory, tokenizer and dataset load through the very calls the script
makes.  The script itself moves the model to CUDA, so its run is a GPU test (tests/test_reference_script_gpu.py)."""
import ast
import subprocess
import sys

import pytest

from tests import reference_env as renv

pytestmark = pytest.mark.skipif(not renv.SCRIPT.exists(), reason="baseline/_ref is empty (python baseline/reference.py --from <checkout>)")


def test_script_imports_and_stand_ins_load(tmp_path):
    env = renv.build(tmp_path)
    tree = ast.parse(renv.SCRIPT.read_text())
    imports = [ast.unparse(node) for node in tree.body
               if isinstance(node, (ast.Import, ast.ImportFrom)) and getattr(node, "module", None) != "__future__"]
    assert any("hybrid_quant.data" in line for line in imports) and any("matplotlib" in line for line in imports)
    code = "\n".join([
        "import sys",
        f"sys.path[:0] = [{str(renv.STUBS)!r}, {str(renv.ROOT)!r}]; sys.path.append({str(renv.REF_DIR)!r})",
        *imports,
        "import hybrid_quant.int4_8b_attention as ia, hybrid_quant.mamba_state_8b_kernel as mk, hybrid_quant.nemotron_8b_decode_eval as ev",
        f"assert ia.__file__.startswith({str(renv.ROOT / 'hybrid_quant')!r}) and mk.__file__.startswith({str(renv.ROOT / 'hybrid_quant')!r})",
        f"assert ev.__file__.startswith({str(renv.REF_DIR)!r}), ev.__file__",
        f"model = AutoModelForCausalLM.from_pretrained({str(env['repo'])!r}, trust_remote_code=True, torch_dtype=torch.bfloat16).eval()",
        f"tokenizer = AutoTokenizer.from_pretrained({str(env['repo'])!r}, trust_remote_code=True)",
        f"texts = load_wikitext_texts({str(env['dataset'])!r}, split='test')",
        "ids = tokenizer('\\n\\n'.join(texts), add_special_tokens=False, return_tensors='pt').input_ids[:, :49]",
        "assert ids.shape == (1, 49) and int(ids.max()) < 511, ids.shape",
        "mamba, attn, mlp = layer_groups(model.config)",
        "assert mamba and attn and mlp and adjacent_mamba_layers(mamba, attn)",
        "patch_attention_cache_in_blocks.__module__",
        "module = __import__(model.__class__.__module__, fromlist=['selective_state_update'])",
        "assert all(hasattr(module, n) for n in ('selective_state_update', 'repeat_kv', 'HybridMambaAttentionDynamicCache'))",
        "cache = module.HybridMambaAttentionDynamicCache(model.config, 1, torch.bfloat16, device=model.device)",
        "out = model(input_ids=ids[:, :8], cache_params=cache, cache_position=torch.arange(8), use_cache=True, return_dict=True)",
        "assert out.logits.shape == (1, 8, 512) and torch.isfinite(out.logits.float()).all()",
        "print('ok')",
    ])
    res = subprocess.run([sys.executable, "-c", code], cwd=tmp_path, env=renv.subprocess_env(tmp_path), capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout[-2000:] + res.stderr[-4000:]
