"""Import-path shim: `import linrec; linrec.linrec(x, c, reverse=...)` keeps working for code
written against safelix/linrec, and resolves to the B200 implementation in `linrec_b200`."""
from linrec_b200 import linrec  # noqa: F401
