"""CPU oracle for the Metis NVFP4 linear-layer path: TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the CPU-baseline legs of bench.py may import this
package; the product (fp4_post_b200) never does.
"""
