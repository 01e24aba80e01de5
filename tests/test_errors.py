"""The error contract: one class per decision, and a code that does not drift.

After the reference's tests/test_errors.py. A host that catches the reference's errors by class,
by builtin base or by code keeps working on this target, so the names, the bases and the codes
are asserted here (the codes are the reference's, ``src/aotolith/errors.py:46-255``).
"""

import inspect

import pytest

import aotolith_b200 as aoto
from aotolith_b200 import errors as E

EXPECTED = {
    "AotolithError": ("AOTO-0000", Exception),
    "CompilationError": ("AOTO-1000", ValueError),
    "UnsupportedOperationError": ("AOTO-1001", NotImplementedError),
    "DynamicShapeError": ("AOTO-1002", ValueError),
    "UnsupportedDTypeError": ("AOTO-1003", ValueError),
    "UnsupportedModelError": ("AOTO-1004", NotImplementedError),
    "IRValidationError": ("AOTO-1010", ValueError),
    "PlanInputError": ("AOTO-2001", ValueError),
    "IndexBoundsError": ("AOTO-2002", IndexError),
    "PlanDTypeError": ("AOTO-2003", TypeError),
    "MemoryBudgetError": ("AOTO-2004", RuntimeError),
    "BucketRangeError": ("AOTO-2005", ValueError),
    "DeviceError": ("AOTO-3001", RuntimeError),
    "ArtifactError": ("AOTO-4001", RuntimeError),
    "ArtifactCompatibilityError": ("AOTO-4002", RuntimeError),
    "PlatformError": ("AOTO-5001", ImportError),
}


def _classes():
    return [cls for _, cls in inspect.getmembers(E, inspect.isclass)
            if issubclass(cls, E.AotolithError) and cls.__module__ == E.__name__]


def test_every_error_is_an_aotolith_error_with_the_reference_code_and_base():
    found = {cls.__name__: cls for cls in _classes()}
    assert set(EXPECTED) <= set(found)
    for name, (code, base) in EXPECTED.items():
        assert found[name].code == code, name
        assert issubclass(found[name], base), name
        assert issubclass(found[name], E.AotolithError)


def test_codes_are_unique_and_well_formed():
    codes = [cls.code for cls in _classes()]
    assert len(codes) == len(set(codes)), "two error classes share a code"
    for code in codes:
        area, _, number = code.partition("-")
        assert area == "AOTO" and len(number) == 4 and number.isdigit(), code


def test_the_refinements_keep_their_parents():
    assert issubclass(E.UnsupportedModelError, E.CompilationError)
    assert issubclass(E.UnsupportedOperationError, E.CompilationError)
    assert issubclass(E.BucketRangeError, E.PlanInputError)
    assert issubclass(E.PlanDTypeError, E.PlanInputError)
    assert issubclass(E.ArtifactCompatibilityError, E.ArtifactError)


def test_a_hint_is_rendered_apart_from_the_message():
    error = E.PlanInputError("expected 2 inputs", hint="pass both")
    assert str(error) == "expected 2 inputs" and error.hint == "pass both"
    assert error.describe() == f"[{E.PlanInputError.code}] expected 2 inputs\nhint: pass both"
    assert E.DeviceError("no device").describe() == "[AOTO-3001] no device"
    assert E.CompilationError("x", code="AOTO-1999").code == "AOTO-1999"       # an instance may refine its code


def test_old_handlers_keep_working():
    with pytest.raises(ValueError):
        raise E.BucketRangeError("too long")
    with pytest.raises(NotImplementedError):
        raise E.UnsupportedModelError("not covered")
    with pytest.raises(IndexError):
        raise E.IndexBoundsError("out of range")
    with pytest.raises(ImportError):
        raise E.PlatformError("no MLX here")


def test_the_public_package_exposes_the_hierarchy():
    for name in EXPECTED:
        assert getattr(aoto, name, None) is getattr(E, name) or getattr(aoto.errors, name) is getattr(E, name)
