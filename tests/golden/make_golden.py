#!/usr/bin/env python3
"""Makes tests/golden/*.npz: what the reference's OWN float64 model computes on
tiny random checkpoints.

The reference's engine (`src/microinfer/model.py`, `engine.py`) cannot be
imported without its CUDA extension and a GPU driver, but its float64 NumPy
model `forward64` (`tools/conditioning.py:43-82`) and its readers
(`src/microinfer/config.py`, `src/microinfer/weights.py`) are plain Python.
This script loads those three from the reference checkout BY PATH, taking
`forward64` out of its file with `ast` (the file's other imports need the
extension), and runs it on the tiny model folders that this library's
random-weights mode writes. It stores, for each tiny configuration, the prompt,
the final-normed hidden states and the logits, plus the SHA-256 of the
model.safetensors it read, so that the test can tell whether the random stream
still produces the same weights.

    python tests/golden/make_golden.py /path/to/reference
"""

import ast
import hashlib
import importlib.util
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))


def load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def reference_forward64(reference: Path):
    config = load_by_path("ref_config", reference / "src/microinfer/config.py")
    weights = load_by_path("ref_weights", reference / "src/microinfer/weights.py")
    source = (reference / "tools/conditioning.py").read_text()
    tree = ast.parse(source)
    wanted = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "forward64"]
    module = ast.Module(body=wanted, type_ignores=[])
    namespace = {"np": np, "Path": Path, "ModelConfig": config.ModelConfig,
                 "read_tensor": weights.read_tensor, "SEED": 0}
    exec(compile(module, "conditioning.py:forward64", "exec"), namespace)
    return config.ModelConfig, weights.read_tensor, namespace["forward64"]


def main(reference):
    from conftest import TINY, prompts_for
    from semantic_aware_adaptive_kv_cache_precision_b200 import write_random_model
    ModelConfig, read_tensor, forward64 = reference_forward64(Path(reference))
    lengths = {"A": 17, "B": 64}
    for name in ("A", "B"):
        config, seed = TINY[name]
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_random_model(Path(tmp) / "m", dict(config), seed, dtype="float32")
            checkpoint = folder / "model.safetensors"
            digest = hashlib.sha256(checkpoint.read_bytes()).hexdigest()
            ids = prompts_for(name, [lengths[name]])[0]
            cfg = ModelConfig.from_dict(name, dict(config))
            states = forward64(cfg, checkpoint, ids, 0.0)
            head = "model.embed_tokens.weight" if config["tie_word_embeddings"] else "lm_head.weight"
            logits = states[-1] @ read_tensor(checkpoint, head).astype(np.float64).T
        keep = np.unique(np.concatenate([np.arange(0, len(ids), 8), [len(ids) - 1]]))
        np.savez_compressed(HERE / f"tiny_{name}.npz", ids=ids, positions=keep,
                            final_hidden=states[-1][keep].astype(np.float32),
                            mid_hidden=states[1][keep].astype(np.float32),
                            logits=logits[keep].astype(np.float32),
                            sha256=np.array(digest))
        print(name, states.shape, logits.shape, digest[:12])


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1
         else str(Path(__file__).resolve().parents[3] / "reference"))
