"""Minimal stand-in for the `aenum` package: only `extend_enum`, which the reference uses to add one
member to an existing `enum.Enum` at import time."""
import enum


def extend_enum(enumeration, name, *args):
    """Add member `name` with value `args[0]` to an existing Enum class."""
    value = args[0] if len(args) == 1 else args
    member = object.__new__(enumeration)
    member._name_ = name
    member._value_ = value
    if hasattr(enumeration, "_member_names_"):
        enumeration._member_names_.append(name)
    enumeration._member_map_[name] = member
    try:
        enumeration._value2member_map_[value] = member
    except TypeError:
        pass
    type.__setattr__(enumeration, name, member)
    return member
