from stk_b200.random.random_ops import dense_mask, mask, randn
