"""crucible_b200: a small, whole inference engine for one NVIDIA B200 (sm_100a).

Everything between a request's tokens and its next token for the Llama-style
dense decoder, built from parts so that another architecture is a matter of
registering its parts and its config.json spelling.
"""
__version__ = "0.1.0"

from .sampling.params import SamplingParams  # noqa: E402,F401


def __getattr__(name):
    # the engine imports torch and needs a GPU; load it on first use only
    if name in ("LLM", "Engine", "EngineOptions", "StepEntry", "Scheduler", "SchedulerOptions",
                "Request"):
        from . import engine as _engine
        from .engine import llm as _llm, scheduler as _sched
        table = {"LLM": _llm.LLM, "Engine": _engine.Engine, "EngineOptions": _engine.EngineOptions,
                 "StepEntry": _engine.StepEntry, "Scheduler": _sched.Scheduler,
                 "SchedulerOptions": _sched.SchedulerOptions, "Request": _sched.Request}
        return table[name]
    raise AttributeError(name)
