"""The reference's own test files, collected from its checkout (see conftest.py)."""
