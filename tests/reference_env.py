"""Runner environment in which the reference's own driver script (``run_nemotron_8b_decode_degradation.py``,
unmodified, from ``baseline/_ref``) runs on this machine: TEST INFRASTRUCTURE.

What the script needs and this image lacks, and what stands in for it (all built under a temporary directory):

* the Nemotron-H-8B checkpoint with its remote modeling code  ->  ``tests/models/nemotron_h_shim`` (config + modeling
  files) with random weights saved beside them, loadable by ``AutoModelForCausalLM.from_pretrained(dir,
  trust_remote_code=True)``;
* its tokenizer  ->  a word-level fast tokenizer over 512 made-up words, loadable by ``AutoTokenizer``;
* WikiText-103  ->  a local dataset directory with a ``wikitext-103-raw-v1`` configuration whose ``test`` split is
  random sequences of those words;
* ``matplotlib``  ->  ``tests/stubs/matplotlib`` (records the series, renders nothing).

``script_command`` builds the command line that runs the script with this repository's ``hybrid_quant`` first on the path
(the two hot-path modules are the library's, everything else falls through to the reference's package), or with the
reference's package alone.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
MODEL_SRC = ROOT / "tests" / "models" / "nemotron_h_shim"
STUBS = ROOT / "tests" / "stubs"
REF_DIR = ROOT / "baseline" / "_ref"
SCRIPT = REF_DIR / "run_nemotron_8b_decode_degradation.py"
VOCAB = 512


def build(tmp: Path, seed: int = 0, n_tokens: int = 4096) -> dict:
    import numpy as np
    import torch

    repo = tmp / "nemotron-h-shim"
    repo.mkdir(parents=True)
    # model: random weights saved beside the config and the modeling files
    from tests.models.nemotron_h_shim import modeling_nemotron_h_shim as shim
    torch.manual_seed(seed)
    model = shim.NemotronHShimForCausalLM(shim.tiny_config()).to(torch.bfloat16)
    model.save_pretrained(repo)
    for name in ("config.json", "configuration_nemotron_h_shim.py", "modeling_nemotron_h_shim.py"):
        shutil.copyfile(MODEL_SRC / name, repo / name)
    # tokenizer: one token per made-up word
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    vocab = {f"w{i}": i for i in range(VOCAB - 1)}
    vocab["<unk>"] = VOCAB - 1
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>").save_pretrained(repo)
    # dataset: a local directory with the configuration name the reference asks for
    import pyarrow as pa
    import pyarrow.parquet as pq
    data = tmp / "wikitext"
    data.mkdir()
    rng = np.random.default_rng(seed)
    lines = [" ".join(f"w{int(i)}" for i in rng.integers(0, VOCAB - 1, size=64)) for _ in range(n_tokens // 64 + 1)]
    pq.write_table(pa.table({"text": lines}), data / "test.parquet")
    (data / "README.md").write_text(
        "---\nconfigs:\n- config_name: wikitext-103-raw-v1\n  data_files:\n  - split: test\n    path: test.parquet\n---\n"
        "Synthetic stand-in for WikiText-103 (random sequences of made-up words).\n")
    return {"repo": repo, "dataset": data, "tmp": tmp}


def subprocess_env(tmp: Path) -> dict:
    """Environment of the script's process: every cache the libraries write goes under ``tmp``."""
    env = dict(os.environ)
    cache = tmp / ".cache"
    env.update(HYBRID_QUANT_CACHE_DIR=str(cache), HF_HOME=str(cache / "hf"), HF_MODULES_CACHE=str(cache / "hf-modules"),
               HF_DATASETS_CACHE=str(cache / "hf" / "datasets"), XDG_CACHE_HOME=str(cache / "xdg"), TRITON_CACHE_DIR=str(cache / "triton"),
               HF_HUB_OFFLINE="1", HF_DATASETS_OFFLINE="1", TRANSFORMERS_OFFLINE="1", TOKENIZERS_PARALLELISM="false")
    env.pop("PYTHONPATH", None)
    return env


def script_command(args: list[str], use_library: bool = True, script: Path = SCRIPT) -> list[str]:
    """``python -c`` command running the reference script unchanged.  ``use_library``: this repository first on the path
    (its ``hybrid_quant`` replaces the two hot-path modules), the reference checkout after it; otherwise the reference's
    package alone (its Triton kernels)."""
    first = [str(STUBS)] + ([str(ROOT)] if use_library else [])
    last = [str(REF_DIR)] + ([] if use_library else [str(ROOT)])  # the model's CUDA baselines need layer_quant_b200 importable
    code = ("import sys, runpy; sys.path[:0] = {first!r}; sys.path.extend({last!r}); sys.argv = {argv!r}; "
            "runpy.run_path({script!r}, run_name='__main__')").format(first=first, last=last, argv=[str(script)] + list(args),
                                                                     script=str(script))
    return [sys.executable, "-c", code]
