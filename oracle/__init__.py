"""TEST INFRASTRUCTURE: CPU oracle of the leaf-parallel evaluation path.

Only tests/, the smoke check and the benchmark's CPU-baseline leg import this
package.  `oracle.capi` wraps liboracle.so (the plain-C restatement) and, when
they were built, the reference project's own classes in oracle/_ref/.
"""
