"""``moeflow`` is an import alias of ``moeflow_b200``: call sites written against the reference's package name
get this framework's modules (the same objects, not copies)."""

import importlib

import pytest


def test_alias_resolves_to_the_same_module_objects():
    import moeflow
    import moeflow.fixed
    import moeflow.reference
    import moeflow_b200.fixed
    import moeflow_b200.reference

    assert moeflow.fixed is moeflow_b200.fixed
    assert moeflow.reference.moe_reference is moeflow_b200.reference.moe_reference
    assert moeflow.MoEConfig is moeflow_b200.MoEConfig and moeflow.GLM53_FLASH is moeflow_b200.GLM53_FLASH
    assert moeflow_b200.fixed.__spec__.name == "moeflow_b200.fixed"  # the real module keeps its own spec


def test_nested_modules_and_unknown_names():
    ops = importlib.import_module("moeflow.integrations.vllm_runner_ops")
    assert ops.__name__ == "moeflow_b200.integrations.vllm_runner_ops"
    with pytest.raises(ImportError):
        importlib.import_module("moeflow.no_such_module")
