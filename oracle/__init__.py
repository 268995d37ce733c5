"""CPU oracle of the decode-time linear operators: TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's CPU-baseline leg import this
package.  The shipped library (adreno-llms_b200/) never does.
"""
