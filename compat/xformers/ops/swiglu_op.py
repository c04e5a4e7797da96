"""Stand-in for xformers.ops.swiglu_op: only the name bench_swiglu.py:8 imports."""


class DualGemmSiluOp:
    @staticmethod
    def OPERATOR(*args, **kwargs):
        raise NotImplementedError("xformers is not installed; this is an import-only stand-in")
