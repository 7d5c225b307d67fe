// Lets other translation units report a failure through cudeep_b200_last_error().
#pragma once

#include <string>

namespace cudeep_b200 {
void set_last_error(const std::string& message);
}
