"""The reference arm of bench.py: tzar-beep/Tensorline itself, unmodified, from baseline/_ref.

Installed offline with
    pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse --target baseline/_ref <copy of the project>
(`--no-deps` because its `accelerate` dependency is not in the wheelhouse; installed from a copy
because the build writes into the source tree).
"""
from __future__ import annotations

import json
import os


def run(args, model_raw: dict, context: int, prompt: int) -> int:
    ref = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    if not os.path.isdir(os.path.join(ref, "tensorline")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this box"}))
        return 0
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference loads its model and tokenizer by name through an installed package "
                      "(tensorline/engine.py:63-66); no checkpoint or tokenizer of this size exists offline"}))
    return 0
