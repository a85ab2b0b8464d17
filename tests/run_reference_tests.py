"""Run one of the reference's own python test files against this package.

    python tests/run_reference_tests.py <path to a test_*.py of the reference>

The reference's tests say ``import mlx.data as dx``; here that name is bound to
this package, nothing else is changed, and the file is loaded from where it
lies.  It runs in a process of its own so that the alias cannot leak into
tests that import the real reference under the same name.  Exit status 0 means
every test in the file passed.
"""
import importlib.util
import os
import sys
import types
import unittest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main(path):
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package

    pkg = load_package()
    alias = types.ModuleType("mlx")
    alias.data = pkg
    sys.modules["mlx"] = alias
    sys.modules["mlx.data"] = pkg
    spec = importlib.util.spec_from_file_location("reference_" + os.path.basename(path)[:-3], path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    suite = unittest.defaultTestLoader.loadTestsFromModule(mod)
    result = unittest.TextTestRunner(stream=sys.stdout, verbosity=2).run(suite)
    print("REFERENCE-TESTS ran=%d failed=%d" % (result.testsRun, len(result.failures) + len(result.errors)))
    return 0 if result.wasSuccessful() and result.testsRun > 0 else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv[1]))
