"""Python surface of the fabric: operand-block packing by queried layouts
(monoserve/fabric/args.py) and lane programs (monoserve/fabric/program.py)."""
