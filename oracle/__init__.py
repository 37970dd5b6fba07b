"""CPU oracle for the triangle-attention / triangle-multiplication path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
folder; only the tests, the smoke entry and the bench's CPU-baseline /
reference legs may call it, and only as the checker or the timed CPU arm.
"""
