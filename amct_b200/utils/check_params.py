"""Argument type checking for the public entry points
(contract of amct_pytorch/utils/check_params.py:24-57: a class argument is
checked with issubclass, anything else with isinstance; TypeError names the
function and the argument)."""
import functools
import inspect

__all__ = ['check_params']


def check_params(**expected):
    def decorate(func):
        sig = inspect.signature(func)

        @functools.wraps(func)
        def wrapper(*args, **kwargs):
            for name, value in sig.bind(*args, **kwargs).arguments.items():
                want = expected.get(name)
                if want is None:
                    continue
                ok = issubclass(value, want) if isinstance(value, type) else isinstance(value, want)
                if not ok:
                    raise TypeError('Func {} argument {} must be {}'.format(func.__name__, name, want))
            return func(*args, **kwargs)

        return wrapper

    return decorate
