"""CPU oracle of Habitat's batched prediction path -- TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
package; the product (habitat_b200) never does.
"""
