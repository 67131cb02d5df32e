"""TEST INFRASTRUCTURE ONLY. CPU oracles for the training step; nothing in the product imports this
package. Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may use it."""
