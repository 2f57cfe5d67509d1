"""``JitConfig``: per-function compile options (python/mindspore/common/jit_config.py).  ``jit_level`` O0 / O1 / O2 and
``exc_mode`` are accepted and stored; the options that change behaviour here are ``debug_level`` (RELEASE / DEBUG: the
latter keeps scope names in the dumped graphs) and ``infer_boost``."""


class JitConfig:
    def __init__(self, jit_level="", exc_mode="auto", jit_syntax_level="", debug_level="RELEASE", infer_boost="off",
                 **kwargs):
        if jit_level not in ("", "O0", "O1", "O2"):
            raise ValueError("For 'jit_level' must be one of '', 'O0', 'O1', 'O2', but got %r" % (jit_level,))
        if exc_mode not in ("auto", "sink", "no_sink"):
            raise ValueError("For 'exc_mode' must be one of 'auto', 'sink', 'no_sink', but got %r" % (exc_mode,))
        if jit_syntax_level not in ("", "STRICT", "COMPATIBLE", "LAX"):
            raise ValueError("For 'jit_syntax_level' must be one of '', 'STRICT', 'COMPATIBLE', 'LAX', but got %r"
                             % (jit_syntax_level,))
        if debug_level not in ("RELEASE", "DEBUG"):
            raise ValueError("For 'debug_level' must be 'RELEASE' or 'DEBUG', but got %r" % (debug_level,))
        if infer_boost not in ("on", "off"):
            raise ValueError("For 'infer_boost' must be 'on' or 'off', but got %r" % (infer_boost,))
        self.jit_config_dict = dict(kwargs)
        self.jit_config_dict.update(jit_level=jit_level, exc_mode=exc_mode, jit_syntax_level=jit_syntax_level,
                                    debug_level=debug_level, infer_boost=infer_boost)

    def __getattr__(self, name):
        d = self.__dict__.get("jit_config_dict", {})
        if name in d:
            return d[name]
        raise AttributeError(name)
