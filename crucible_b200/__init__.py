"""crucible_b200: a small, whole inference engine for one NVIDIA B200 (sm_100a).

Everything between a request's tokens and its next token for the Llama-style
dense decoder, built from parts so that another architecture is a matter of
registering its parts and its config.json spelling.
"""
__version__ = "0.1.0"
