"""CPU oracle (test infrastructure): a C restatement of the reference's CPU references.

Only the test-suite, the smoke entry and the benchmark's CPU-baseline leg may import this
package.  The product library never does.
"""
