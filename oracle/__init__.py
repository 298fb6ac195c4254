"""TEST INFRASTRUCTURE -- the CPU oracle.  Not part of the shipped library.

A plain-torch restatement of the reference HIR evaluator's arithmetic for the
decode step: one torch call per HIR op at the declared dtype, following each
authored ``@func`` body line by line.  Only ``tests/``, ``__graft_entry__.smoke``
and the CPU-baseline / reference legs of ``bench.py`` may import this package;
nothing under ``tilefoundry_b200/`` does.

Why a restatement: the reference package cannot be imported without isl-python,
ortools and graphviz (its parser builds isl maps while type-checking a function),
none of which is installed or installable offline.  The arithmetic itself lives in
PyTorch, which is present, so calling the same torch ops in the same order
reproduces the evaluator's values.

Pinning: the reference holds no numeric golden vectors; its own tests pin the
authored models against seeded Hugging Face modules
(``tests/models/decode_oracle.py:126-137,213-233``).  ``tests/golden/`` holds
vectors generated the same way here (script committed beside them) and
``tests/test_oracle_pins.py`` checks this oracle against them and against the
reference's own importable torch transcriptions.
"""
