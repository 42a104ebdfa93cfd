"""Parity checker (test infrastructure).  Never imported by the product package."""
