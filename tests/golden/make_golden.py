"""Runs the reference's own GPT-2 (``rosellm.rosetrainer.model.GPTModel``) on the CPU for the
tiny test models and stores its logits beside this script.

    python tests/golden/make_golden.py --reference PATH_TO_ROSELLM_CHECKOUT

The tiny model folders are written by the package's random-weights mode, renamed for the
reference by the reference's own ``convert_hf_gpt2_state_dict``.  The reference never reads
``layer_norm_epsilon`` (every LayerNorm keeps torch's default), so the ``eps`` attribute of
its LayerNorm modules is set after construction.  ``tests/test_plain_cpu.py`` checks the plain
implementation against the stored logits; the script also prints the difference it sees.
"""
import argparse
import hashlib
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import plain_gpt2 as P  # noqa: E402
from tiny import TINY, write_tiny  # noqa: E402

SEQ_LEN = {"A": 24, "B": 31}


def weights_digest(tensors: dict) -> str:
    h = hashlib.sha256()
    for k in sorted(tensors):
        h.update(k.encode())
        h.update(tensors[k].to(torch.float32).numpy().tobytes())
    return h.hexdigest()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of chtho-like/rosellm")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from rosellm.rosetrainer.config import GPTConfig
    from rosellm.rosetrainer.hf_gpt2 import convert_hf_gpt2_state_dict
    from rosellm.rosetrainer.model import GPTModel

    root = tempfile.mkdtemp()
    for name in ("A", "B"):
        folder = write_tiny(name, root)
        cfg, t = P.load_folder(folder, torch.float32)
        ref_cfg = GPTConfig(
            vocab_size=cfg["vocab_size"], max_position_embeddings=cfg["n_positions"], n_layers=cfg["n_layer"],
            n_heads=cfg["n_head"], d_model=cfg["n_embd"], d_ff=cfg["n_inner"], dropout=0.0,
            activation=cfg["activation_function"],
        )
        model = GPTModel(ref_cfg).eval()
        mapped = convert_hf_gpt2_state_dict({"transformer." + k: v for k, v in t.items()}, n_layers=cfg["n_layer"])
        model.load_state_dict(mapped, strict=True)
        for m in model.modules():
            if isinstance(m, torch.nn.LayerNorm):
                m.eps = cfg["layer_norm_epsilon"]
        ids = torch.from_numpy(np.random.default_rng(100 + len(name)).integers(0, cfg["vocab_size"], SEQ_LEN[name]))
        with torch.no_grad():
            logits, _ = model(ids[None, :])
        logits = logits[0].float().numpy()
        cfg64, t64 = P.load_folder(folder)
        mine = P.forward(cfg64, t64, ids).numpy()
        print(f"tiny {name}: reference logits {logits.shape}, max|plain - reference| = {np.abs(mine - logits).max():.3e}, "
              f"max|logit| = {np.abs(logits).max():.3f}")
        np.savez_compressed(os.path.join(HERE, f"tiny_{name}.npz"), ids=ids.numpy(), logits=logits,
                            weights_sha256=np.array(weights_digest(t)))


if __name__ == "__main__":
    main()
