"""CPU oracle for the attention / KV-cache Monte-Carlo decode path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this
directory; it is the checker the parity tests, the smoke run and the CPU
baseline leg of the benchmark compare against.
"""
