def split_key(key: str) -> list[str]:
    """'a.b[0].c' -> ['a', 'b', '0', 'c'] (the dotted / bracketed key grammar of omegaconf)."""
    out, cur, i = [], "", 0
    while i < len(key):
        ch = key[i]
        if ch == ".":
            if cur or not out:
                out.append(cur)
            cur = ""
        elif ch == "[":
            if cur:
                out.append(cur)
            j = key.index("]", i)
            out.append(key[i + 1:j])
            cur = ""
            i = j
        else:
            cur += ch
        i += 1
    if cur:
        out.append(cur)
    return out
