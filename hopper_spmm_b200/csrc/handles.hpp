// The opaque host-side handles of the C ABI, shared by the translation units that implement it.
#pragma once

#include "format.hpp"
#include "formats_ext.hpp"

struct b200spmm_btcf {
    b200spmm::Btcf f;
};

struct b200spmm_btcfb {
    b200spmm::BtcfBitmap f;
};

struct b200spmm_gbtcf {
    b200spmm::Gbtcf g;
};

struct b200spmm_csr {
    b200spmm::CsrHost m;
};
