"""flyingfish_b200: a Blackwell-native (sm_100a) LLM inference engine.

Public surface: :class:`flyingfish_b200.api.Model` (load / prefill / decode / generate),
the ``ff`` command line (:mod:`flyingfish_b200.cli`) and the OpenAI-compatible server
(:mod:`flyingfish_b200.serve`).
"""
__version__ = "0.1.0"
