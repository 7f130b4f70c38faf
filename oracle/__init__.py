"""CPU oracle for the joint-attention path.  Test infrastructure only: nothing in the product imports it."""
