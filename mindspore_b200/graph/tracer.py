"""Trace state shared by Primitive, GradOperation and the jit front end (filled in by graph.jit)."""
_current = None


def is_tracing():
    return _current is not None


def current():
    return _current


def _set_current(t):
    global _current
    _current = t
