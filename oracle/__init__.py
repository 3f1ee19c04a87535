"""CPU oracle of the gpt_lm hot path. TEST INFRASTRUCTURE ONLY: imported by tests/, by
__graft_entry__.smoke() and by bench.py's CPU-baseline / reference arms, never by the product
package."""
