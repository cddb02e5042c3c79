"""Choice of the bfloat16 flash attention kernel (filled in as the kernel lands)."""


def run(q, k_pages, v_pages, block_table, out, H, G, hd, page_tokens, window, scale, plan) -> bool:
    return False
