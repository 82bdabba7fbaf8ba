"""imparo_b200: a small, whole inference engine for one B200, built from what
zeraix/imparo shows.  Public entry points: Engine (Python), `python -m imparo_b200` (command
line), bin/trace_run (replay of given tokens)."""
__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "StepItem"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
