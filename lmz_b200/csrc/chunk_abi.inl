// chunk ABI
