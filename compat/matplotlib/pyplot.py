"""No-op pyplot: every call is accepted and ignored."""


class _Noop:
    def __getattr__(self, name):
        return self

    def __call__(self, *args, **kwargs):
        return self

    def __iter__(self):
        return iter(())


_noop = _Noop()


def figure(*a, **k):
    return _noop


def subplot(*a, **k):
    return _noop


def subplots(*a, **k):
    return _noop, _noop


def __getattr__(name):
    return _noop
