"""CPU checkers (test infrastructure, never on a product path).

`oracle.sgref`  -- this repository's C restatement of the reference arithmetic (sgref.c).
`oracle.refapi` -- the unmodified reference library compiled from its own sources into oracle/_ref/.
Only tests/, the smoke check and the CPU-baseline legs of bench.py import this package.
"""
