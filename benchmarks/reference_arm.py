"""Reference arm of bench.py (filled in once the reference is installed under baseline/_ref)."""
import json


def run_reference(args):
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired yet"}))
