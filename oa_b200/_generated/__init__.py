"""Tables written by oa_b200.devtools.autogen (checked against their generators by the drift gate)."""
