"""Reference arm of ``bench.py``: runs the unmodified reference project for the headline config,
or reports in one line why it cannot run on this machine."""
from __future__ import annotations

import importlib.util
import os

ROOT = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(ROOT, "_ref")


def _missing(mods):
    return [m for m in mods if importlib.util.find_spec(m) is None]


def run(args) -> dict:
    """Returns the JSON-able result dict of the reference run (or ``{"unavailable": why}``)."""
    base = {"impl": "reference", "n_gpus": args.gpus}
    if not os.path.isdir(os.path.join(REF_DIR, "hmf")):
        base["unavailable"] = ("reference package not installed under baseline/_ref: its build backend (hatchling) "
                               "is absent offline and pip cannot build it")
        return base
    need = _missing(["deepspeed", "accelerate", "peft", "trl", "omegaconf", "mamba_ssm", "causal_conv1d"])
    if need:
        base["unavailable"] = ("reference `hmf train` cannot import here: missing " + ", ".join(need) +
                               " (no network, not in the offline wheelhouse)")
        return base
    base["unavailable"] = "reference runner not wired for this configuration"
    return base
