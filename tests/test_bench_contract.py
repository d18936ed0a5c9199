"""What bench.py answers without a GPU: the reference arm and a request for several GPUs."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True,
                          text=True, timeout=120)


def test_reference_arm_says_why_it_is_unavailable():
    out = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3")
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_more_than_one_gpu_is_one_line_and_exit_code_two():
    out = _run("--gpus", "2", "--steps", "2", "--warmup", "3")
    assert out.returncode == 2
    assert len(out.stdout.strip().splitlines()) == 1 and "one GPU" in out.stdout


def test_design_option_builds_layers_of_equal_size():
    """The option that sets Zededra layers beside the dense decoder: its configurations
    parse, and the two arms hold the same width, heads, feed-forward and cache bytes a token."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("design_bench", ROOT / "baseline" / "design_bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    from mini_llm_stack_b200.config import config_from_dict
    assert "--design" in _run("--help").stdout
    for s in mod.SIZES.values():
        dense = config_from_dict(mod.llama_config(s, 2))
        for kind in ("latent_dense", "latent_moe", "mlstm_dense"):
            z = config_from_dict(mod.zededra_config(s, kind, 2))
            assert z.width == dense.d_model and len(z.layers) == dense.n_layers
        latent = mod.zededra_config(s, "latent_dense", 2)["layers"][0]
        assert latent["mixer"]["heads"] == dense.n_heads and latent["mlp"]["ff"] == dense.intermediate_size
        assert 2 * dense.n_kv_heads * dense.head_dim >= latent["mixer"]["kv_rank"]
        for kind in mod.DESIGNS["logulix"][1]:
            g = config_from_dict(mod.logulix_config(s, kind, 2))
            assert g.width == dense.d_model and len(g.layers) == dense.n_layers
            assert g.layers[0]["mlp"]["ff"] == dense.intermediate_size
        att = mod.logulix_config(s, "attention_dense", 2)["layers"][0]["mixer"]
        assert (att["heads"], att["kv_heads"], att["dim"]) == (dense.n_heads, dense.n_kv_heads,
                                                               dense.head_dim)
        for kind in mod.DESIGNS["movazen"][1]:
            m = config_from_dict(mod.movazen_config(s, kind, 2))
            assert m.width == dense.d_model and len(m.layers) == dense.n_layers
        att = mod.movazen_config(s, "attention_moe", 2)["layers"][0]["mixer"]
        assert (att["heads"], att["kv_heads"], att["dim"]) == (dense.n_heads, dense.n_kv_heads,
                                                               dense.head_dim)
        moe = mod.movazen_config(s, "parallel_moe", 2)["layers"][0]["mlp"]
        assert (moe["router"]["experts"], moe["router"]["top"], moe["expert"]["ff"]) == \
            (s["experts"], s["top"], s["eff"])
