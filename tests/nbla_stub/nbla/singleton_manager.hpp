#include <nbla/stub_core.hpp>
