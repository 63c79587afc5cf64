"""CPU oracle of the model-forward path. TEST INFRASTRUCTURE ONLY.

Nothing under ``oracle/`` is part of the product: only ``tests/``, ``__graft_entry__.smoke()``
and ``bench.py``'s CPU-baseline / reference legs may import it, as the checker or the timed
CPU baseline. The package under ``infinity_b200/`` never imports it.

Parity status: the reference's forward lives in third-party packages that are not in the
reference tree (sentence-transformers 3.3.1, transformers 4.47.0, torch 2.8.0 per its
lock file) and needs hub checkpoints; none of its numeric pins can run offline. The
encoder restatement is therefore pinned against the locally installed ``transformers``
model classes the reference would call (see ``tests/test_oracle.py``), and pooling /
normalisation against golden vectors produced by the reference's own numpy code
(``tests/golden``). Forward numerics against the reference's exact pinned versions:
PARITY UNPINNED.
"""
