"""Framework adapters.  Each sub-package registers one adapter; absent frameworks simply never detect."""
