"""Accounting and checking helpers: parameter / FLOP counts and the numeric pass-fail rule of value checks."""
