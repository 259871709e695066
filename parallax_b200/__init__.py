"""parallax_b200 — a Blackwell-native pipeline-parallel LLM serving engine.

Public surface: the ``parallax`` CLI (``serve``, ``run``, ``join``, ``chat``), the
OpenAI-compatible HTTP frontend, the cluster scheduler / router, and the in-process
``Engine`` used by the benchmarks.
"""

__version__ = "0.1.0"
