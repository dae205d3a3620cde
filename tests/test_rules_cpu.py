"""The by-name launch table: names, parameter lists in the reference's order, and refusals before any launch."""
import pytest


def test_table_lists_the_reference_parameters():
    from tessera_b200 import rules
    assert rules.RULES["attend_rows"].params == ("q", "k", "v", "out", "slots", "positions", "rows", "keys", "heads",
                                                 "kv_heads", "width", "back")   # attend.rs:126-139
    assert rules.RULES["scatter"].params == ("x", "slots", "positions", "out", "rows", "width")   # scatter.rs:12-19
    assert rules.RULES["top_k"].params == ("x", "out", "rows", "width", "k")   # argmax.rs:39
    assert rules.RULES["lane_norm"].params == ("x", "w", "out", "rows", "width", "eps")   # lane_norm.rs:10-17
    for name in ("lanes", "thin", "tiled"):
        assert rules.RULES[name].params == ("x", "w", "out", "n", "k")
    assert all(r.cites.startswith("engine/") for r in rules.RULES.values())


def test_unknown_names_and_wrong_counts_are_refused():
    from tessera_b200 import rules
    with pytest.raises(KeyError):
        rules.launch("no_such_kernel", [])
    with pytest.raises(TypeError):
        rules.launch("top_k", [1, 2, 3])
