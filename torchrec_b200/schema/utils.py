"""Backward-compatibility check of public signatures (``torchrec/schema/utils.py:38``): a new signature is compatible when every
call that was valid against the old one stays valid."""
from __future__ import annotations

import inspect
import typing
from typing import Any


def _is_annot_compatible(prev: object, curr: object) -> bool:
    if prev == curr or prev is inspect.Parameter.empty or curr is inspect.Parameter.empty:
        return True
    if not (prev_origin := typing.get_origin(prev)):
        # a plain type may widen into Optional / Union that contains it
        return typing.get_origin(curr) is typing.Union and prev in typing.get_args(curr)
    curr_origin = typing.get_origin(curr)
    if prev_origin is typing.Union and curr_origin is typing.Union:
        return all(any(_is_annot_compatible(p, c) for c in typing.get_args(curr)) for p in typing.get_args(prev))
    if prev_origin != curr_origin:
        return False
    pa, ca = typing.get_args(prev), typing.get_args(curr)
    if len(pa) != len(ca):
        return False
    return all(_is_annot_compatible(p, c) for p, c in zip(pa, ca))


def is_signature_compatible(previous_signature: inspect.Signature, current_signature: inspect.Signature) -> bool:
    prev = list(previous_signature.parameters.values())
    curr = list(current_signature.parameters.values())
    by_name = {p.name: p for p in curr}
    has_var_pos = any(p.kind == p.VAR_POSITIONAL for p in curr)
    has_var_kw = any(p.kind == p.VAR_KEYWORD for p in curr)
    # positional parameters keep their place and name
    prev_pos = [p for p in prev if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    curr_pos = [p for p in curr if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    for i, p in enumerate(prev_pos):
        if i >= len(curr_pos):
            if not has_var_pos:
                return False
            continue
        c = curr_pos[i]
        if c.name != p.name and p.kind != p.POSITIONAL_ONLY:
            return False
        if p.default is not p.empty and c.default is p.empty:
            return False
        if not _is_annot_compatible(p.annotation, c.annotation):
            return False
    # keyword-only parameters still exist (or are swallowed by **kwargs)
    for p in prev:
        if p.kind == p.KEYWORD_ONLY:
            c = by_name.get(p.name)
            if c is None:
                if not has_var_kw:
                    return False
                continue
            if p.default is not p.empty and c.default is p.empty:
                return False
            if not _is_annot_compatible(p.annotation, c.annotation):
                return False
        if p.kind == p.VAR_POSITIONAL and not has_var_pos:
            return False
        if p.kind == p.VAR_KEYWORD and not has_var_kw:
            return False
    # anything new must be optional
    prev_names = {p.name for p in prev}
    for i, c in enumerate(curr):
        if c.name in prev_names or c.kind in (c.VAR_POSITIONAL, c.VAR_KEYWORD):
            continue
        if c.kind in (c.POSITIONAL_ONLY, c.POSITIONAL_OR_KEYWORD) and i < len(prev_pos):
            continue  # renamed positional-only handled above
        if c.default is c.empty:
            return False
    return _is_annot_compatible(previous_signature.return_annotation, current_signature.return_annotation)
