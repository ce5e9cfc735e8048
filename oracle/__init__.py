"""CPU oracle for the GradCraft training hot path (test infrastructure, never on the product path).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference legs may import this
package.  The CUDA library never calls into it and has no CPU fallback.
"""
